// Launchers of the element-wise / recurrent / attention kernels that sit between the
// weight-streaming GEMMs of one verify or draft pass.  All of them work on the whole block
// of <= 16 token rows at once and never touch the host.
#pragma once
#include "gemm_ts.cuh"

namespace dfl {

#ifdef __CUDACC__
// Packs four consecutive columns k..k+3 (k % 4 == 0, inside one 256-column block) of one
// token row into the activation chunk the few-row GEMM consumes.
__device__ __forceinline__ void pack_quad(uint8_t* chunk, bool bf3, int tok, int k, const float (&v)[4], bool& overflow) {
    const int pos = act_pos(k);
    if (!bf3) {
        uint16_t hi[4], lo[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float f = v[e];
            overflow |= (fabsf(f) >= 65504.f) && (fabsf(f) < INFINITY);
            const __half h = __float2half_rn(f);
            hi[e] = __half_as_ushort(h);
            lo[e] = __half_as_ushort(__float2half_rn(f - __half2float(h)));
        }
        *reinterpret_cast<uint2*>(chunk + (tok * ACT_ROW_HALFS + pos) * 2) =
            make_uint2((uint32_t)hi[0] | ((uint32_t)hi[1] << 16), (uint32_t)hi[2] | ((uint32_t)hi[3] << 16));
        *reinterpret_cast<uint2*>(chunk + ACT_PLANE + (tok * ACT_ROW_HALFS + pos) * 2) =
            make_uint2((uint32_t)lo[0] | ((uint32_t)lo[1] << 16), (uint32_t)lo[2] | ((uint32_t)lo[3] << 16));
    } else {
        uint16_t b[3][4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float f = v[e];
#pragma unroll
            for (int p = 0; p < 3; ++p) {
                const __nv_bfloat16 h = __float2bfloat16_rn(f);
                b[p][e] = __bfloat16_as_ushort(h);
                f -= __bfloat162float(h);
            }
        }
#pragma unroll
        for (int p = 0; p < 3; ++p)
            *reinterpret_cast<uint2*>(chunk + p * ACT_PLANE + (tok * ACT_ROW_HALFS + pos) * 2) =
                make_uint2((uint32_t)b[p][0] | ((uint32_t)b[p][1] << 16), (uint32_t)b[p][2] | ((uint32_t)b[p][3] << 16));
    }
}
// Layout-agnostic forms: `layout` is ACT_F16, ACT_BF3 or ACT_TS (the kernel family of the consuming GEMM).
__device__ __forceinline__ int act_chunk_dev(int layout) {
    return layout == ACT_TS ? ACTTS_CHUNK : layout == ACT_TSB ? ACTTSB_CHUNK : layout == ACT_BF3 ? ACTB3_CHUNK : ACT16_CHUNK;
}
__device__ __forceinline__ void pack_quad_any(uint8_t* chunk, int layout, int tok, int k, const float (&v)[4], bool& overflow) {
    if (layout == ACT_TS) pack_quad_ts(chunk, tok, k, v, overflow);
    else if (layout == ACT_TSB) pack_quad_tsb(chunk, tok, k, v);
    else pack_quad(chunk, layout == ACT_BF3, tok, k, v, overflow);
}
// sum of one token's activations over the 32-column sub-block `sub` (the K-quant "min" term input)
__device__ __forceinline__ void store_subsum(uint8_t* chunk, int layout, int tok, int sub, float sum, bool& overflow) {
    if (layout == ACT_F16) reinterpret_cast<float*>(chunk + 2 * ACT_PLANE)[tok * 8 + sub] = sum;
    else if (layout == ACT_TS) pack_subsum_ts(chunk, tok, sub, sum, overflow);
}
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) {
    if (x > 20.0f) return x;
    if (x < -20.0f) return expf(x);
    return logf(1.0f + expf(x));
}
#endif

constexpr int GLUE_COLS = 64;  // columns per glue CTA = granularity of the sum-of-squares partials

enum GlueMode : int {
    GLUE_RESID = 0,   // v = x + sum_s part[s]        (x updated in place when x != nullptr)
    GLUE_SWIGLU = 1,  // v = silu(sum part[:, c]) * sum part[:, F + c]
    GLUE_COPY = 2     // v = x (read only)
};

struct GlueParams {
    int mode = GLUE_RESID;
    const float* part = nullptr;  // [splits][16][ld_part]
    int splits = 0;
    const int32_t* splits_dev = nullptr;   // optional: *splits_dev more slices follow the first `splits` (a device-chosen count)
    int ld_part = 0;
    float* x = nullptr;           // [16][ld_x]
    int ld_x = 0;
    const float* mul_w = nullptr; // per-column multiplier (a folded RMSNorm weight)
    float pre_scale = 1.f;
    uint8_t* acts = nullptr;      // packed output, optional
    int bf3 = 0;
    float* xn = nullptr;          // optional f32 copy of the packed value [16][ld_xn]
    int ld_xn = 0;
    float* sumsq = nullptr;       // optional [k / GLUE_COLS][16] partial sums of v*v
    float* capture = nullptr;     // optional copy of v: capture[tok * ld_capture + col]
    int ld_capture = 0;
    int swiglu_f = 0;
    // routed experts (GLUE_SWIGLU only): column c < route_e * route_f belongs to expert c / route_f and is
    // multiplied by route_w[tok][expert]; the columns after them (the shared expert) by route_sg[tok]
    const float* route_w = nullptr;
    const float* route_sg = nullptr;
    int route_e = 0, route_f = 0;
    int route_e0 = 0, route_n = 0;   // the inner columns hold experts route_e0 .. route_e0 + route_n - 1
    int n_rows = 0;
    int* err = nullptr;
};
#ifdef __CUDACC__
// The glue of one (token, four consecutive columns) item: columns 64 cb + 4 quad .. + 3 of token `tok`.  The 32 lanes of
// the calling warp must be two tokens x the sixteen quads of one 64-column block (lane = 16 (tok & 1) + quad): the sum
// of squares is reduced over a token's 16 lanes and the 32-column sub-block sums over 8 lanes.
__device__ __forceinline__ void glue_quad(const GlueParams& p, int n_splits, int cb, int tok, int quad) {
    const int col0 = cb * GLUE_COLS + quad * 4;
    const bool live = tok < p.n_rows;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (live) {
        if (p.mode == GLUE_SWIGLU) {
            // route weight of this row for the expert the columns belong to (1 without routing); a row that did not
            // choose the expert gets exact zeros and its partial sums - possibly stale - are not even read
            float w = 1.f;
            if (p.route_w) w = col0 < p.route_n * p.route_f ? p.route_w[tok * p.route_e + p.route_e0 + col0 / p.route_f] : p.route_sg[tok];
            if (w != 0.f) {
                float g[4] = {0.f, 0.f, 0.f, 0.f}, u[4] = {0.f, 0.f, 0.f, 0.f};
                const float* base = p.part + (uint64_t)tok * p.ld_part + col0;
                const uint64_t stride = (uint64_t)MAX_ROWS * p.ld_part;
#pragma unroll 4
                for (int s = 0; s < n_splits; ++s) {
                    const float4 a = __ldcg(reinterpret_cast<const float4*>(base + s * stride));
                    const float4 b = __ldcg(reinterpret_cast<const float4*>(base + s * stride + p.swiglu_f));
                    g[0] += a.x; g[1] += a.y; g[2] += a.z; g[3] += a.w;
                    u[0] += b.x; u[1] += b.y; u[2] += b.z; u[3] += b.w;
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) v[j] = silu_f(g[j]) * u[j];
                if (p.route_w) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) v[j] *= w;
                }
            }
        } else {
            float4 xv = make_float4(0.f, 0.f, 0.f, 0.f);
            if (p.x) xv = *reinterpret_cast<const float4*>(p.x + (uint64_t)tok * p.ld_x + col0);
            if (p.mode == GLUE_RESID && p.part) {
                // sum the split-K partials first (fixed order), then add to the residual
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
                const float* base = p.part + (uint64_t)tok * p.ld_part + col0;
                const uint64_t stride = (uint64_t)MAX_ROWS * p.ld_part;
#pragma unroll 4
                for (int s = 0; s < n_splits; ++s) {
                    const float4 a = __ldcg(reinterpret_cast<const float4*>(base + s * stride));
                    acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
                }
                v[0] = xv.x + acc[0]; v[1] = xv.y + acc[1]; v[2] = xv.z + acc[2]; v[3] = xv.w + acc[3];
                if (p.x) *reinterpret_cast<float4*>(p.x + (uint64_t)tok * p.ld_x + col0) = make_float4(v[0], v[1], v[2], v[3]);
            } else {
                v[0] = xv.x; v[1] = xv.y; v[2] = xv.z; v[3] = xv.w;
            }
        }
        if (p.capture)
            *reinterpret_cast<float4*>(p.capture + (uint64_t)tok * p.ld_capture + col0) = make_float4(v[0], v[1], v[2], v[3]);
    }
    if (p.sumsq) {
        float ss = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (quad == 0) p.sumsq[cb * MAX_ROWS + tok] = ss;
    }
    if (p.mul_w) {
        const float4 w = *reinterpret_cast<const float4*>(p.mul_w + col0);
        v[0] *= w.x; v[1] *= w.y; v[2] *= w.z; v[3] *= w.w;
    }
    if (p.pre_scale != 1.f) {
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] *= p.pre_scale;
    }
    if (p.xn && live) *reinterpret_cast<float4*>(p.xn + (uint64_t)tok * p.ld_xn + col0) = make_float4(v[0], v[1], v[2], v[3]);
    if (p.acts) {
        uint8_t* chunk = p.acts + (uint64_t)(col0 >> 8) * act_chunk_dev(p.bf3);
        bool over = false;
        pack_quad_any(chunk, p.bf3, tok, col0 & 255, v, over);
        if ((p.bf3 == ACT_F16 || p.bf3 == ACT_TS)) {
            float sum = v[0] + v[1] + v[2] + v[3];  // 32-column sub-block = eight neighbouring threads
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            if ((quad & 7) == 0) store_subsum(chunk, p.bf3, tok, (col0 & 255) >> 5, sum, over);
        }
        if (over) atomicCAS(p.err, 0, DEV_ERR_OVERFLOW);
    }
}
#endif
// k = number of columns (multiple of 256)
dfl_status launch_glue(cudaStream_t st, const GlueParams& p, uint64_t k);
// Softmax + top-k routing of n_rows tokens over n_expert experts; logits[tok][n_expert] is the extra router row of
// the shared expert's gate.  Writes route_w[16][n_expert] (zeros for experts not chosen), shared_gate[16],
// route_idx[16][n_used].
// A NaN / Inf logit in a row leaves that row unrouted and sets DEV_ERR_NONFINITE in *err (the reference's NONFINITE route status).
dfl_status launch_moe_route(cudaStream_t st, const float* logits, int ld, int n_expert, int n_used, int n_rows, float* route_w,
                            float* shared_gate, int32_t* route_idx, int* err);
// routing and the lists below in one launch (moe_route_lists_fused says whether the expert count allows it)
bool moe_route_lists_fused(int n_expert);
dfl_status launch_moe_route_lists(cudaStream_t st, const float* logits, int ld, int n_expert, int n_used, int n_rows, float* route_w,
                                  float* shared_gate, int32_t* route_idx, int e0, int n_local, int tiles_per_expert, int shared_tiles,
                                  int min_tiles, int32_t* tile_map, int32_t* n_tiles, int kb_per_expert, int min_kb, int32_t* kb_map,
                                  int32_t* n_kb, int kc, int down_tiles, int max_splits, int* err);
// row tiles of the gate|up matrix that belong to experts some row of the block chose (plus the shared expert)
dfl_status launch_moe_tiles(cudaStream_t st, const float* route_w, int n_rows, int n_expert, int e0, int n_local, int tiles_per_expert,
                            int shared_tiles, int min_tiles, int32_t* tile_map, int32_t* n_tiles, int kb_per_expert, int min_kb, int32_t* kb_map,
                            int32_t* n_kb, int kc, int down_tiles, int max_splits);

// x[tok][0..h) = decoded row tokens[tok] of a ggml matrix [vocab][h] (kernel_get_rows_*,
// kernels/elementwise.metal:727-958).  tokens live on the device.
dfl_status launch_embed_rows(cudaStream_t st, int dtype, const uint8_t* ggml, uint64_t h, const int32_t* tokens, int n_rows,
                             float* x, int ld);

// out[tok][j] = rs[tok] * sum_k xn[tok][k] * w[j][k] for small f32 matrices (GDN alpha/beta, MoE router).
dfl_status launch_small_matmul(cudaStream_t st, const float* w, const float* xn, int ld_xn, int n_rows, uint64_t k, int n_out,
                               const GemmEpilogue& ep, float* out, int ld_out);

// ---- attention (attn.cu) -------------------------------------------------------
struct AttnGeom {
    int n_q, n_kv, hd, n_rot;
    float theta, eps;
};
constexpr int ATTN_CHUNK = 64;
constexpr int ATTN_ROW_GROUP = 4;  // query rows per attention CTA
// KV cache storage: position-major rows [pos][n_kv][hd] of f32 or f16, or (f16, 128-wide heads) tiles of 128 positions
// per KV head in the operand layout of tcgen05.mma (attn_t5.cu)
enum KvMode { KV_F32_ROWS = 0, KV_F16_ROWS = 1, KV_F16_TILED = 2 };
constexpr int KV_TILE_KEYS = 128;
// element index (in halfs) of a tile and of (key, dim) inside a K tile (B[n = key][k = dim]) and a V tile (B[n = dim][k = key]):
// 8 x 8 core matrices of 64 halfs, the sixteen n-groups of a k-core contiguous, k-cores 1024 halfs apart
__host__ __device__ inline uint64_t kv_tile_base(uint32_t pos, int n_kv, int h) { return ((uint64_t)(pos / KV_TILE_KEYS) * n_kv + h) * (uint64_t)(KV_TILE_KEYS * 128); }
__host__ __device__ inline uint32_t kv_tile_k_off(uint32_t key, int d) { return (uint32_t)((d >> 3) * 1024 + (int)(key >> 3) * 64 + (int)(key & 7) * 8 + (d & 7)); }
__host__ __device__ inline uint32_t kv_tile_v_off(uint32_t key, int d) { return (uint32_t)((int)(key >> 3) * 1024 + (d >> 3) * 64 + (d & 7) * 8 + (int)(key & 7)); }
// Reduces the fused q|k|v GEMM partials, applies per-head RMSNorm + partial NeoX RoPE, appends K/V
// at positions start..start+n_rows-1 and leaves rotated Q and the raw gate for the attention kernel.
// gated: q rows are interleaved (q, gate) per head as in the target; otherwise plain q.
// pos_override[tok] (device) replaces start + tok as the RoPE position; cache_row0 >= 0 stores
// K/V at rows cache_row0 + tok instead of at the position (the drafter's context cache).
dfl_status launch_attn_front(cudaStream_t st, const AttnGeom& g, bool gated, const float* part, int splits, int ld_part,
                             const float* q_norm_w, const float* k_norm_w, uint32_t start, int n_rows, void* k_cache,
                             void* v_cache, int kv_mode, float* q_rot, float* gate, const uint32_t* pos_override,
                             long long cache_row0 = -1);
// Causal attention of the n_rows query rows over cache positions [0, start + row]; partials per
// 64-position chunk, then combine, sigmoid gate and activation packing for the o-projection.
dfl_status launch_attn_verify(cudaStream_t st, const AttnGeom& g, const float* q_rot, const float* gate, const void* k_cache,
                              const void* v_cache, int kv_mode, uint32_t start, int n_rows, float* partials, uint8_t* acts,
                              int act_layout, float* out_f32, int* err, uint32_t kv_capacity = 0);
// tcgen05 span kernel over a tiled fp16 cache (attn_t5.cu) and the conversions between that cache and position-major rows
bool attn_t5_supported(const AttnGeom& g, bool kv_f16);
int attn_t5_chunks_per_span(const AttnGeom& g, uint32_t kv_capacity);
dfl_status launch_attn_t5(cudaStream_t st, const AttnGeom& g, const float* q_rot, const void* k_cache, const void* v_cache, uint32_t start,
                          int n_rows, float* partials, int chunks_per_span, int* err);
// rows of logits ordered for the host sampler (sortrows.cu)
uint64_t sort_rows_scratch_bytes(int n_rows, uint64_t vocab);
dfl_status launch_sort_rows_desc(cudaStream_t st, const float* logits, int n_rows, uint64_t vocab, uint64_t ld, void* scratch, uint32_t* order);
// the drafter's attention over a tiled hi + lo shadow of its f32 context cache (attn_t5.cu)
uint64_t dattn_t5_tile_halfs(int n_kv, uint32_t n_keys);
dfl_status launch_dctx_tiles(cudaStream_t st, const float* k_rows, const float* v_rows, int n_kv, uint32_t first, uint32_t count, uint32_t row0,
                             void* tiles);
dfl_status launch_dattn_t5(cudaStream_t st, const AttnGeom& g, const float* q_rot, const void* ctx_tiles, const void* noise_tiles,
                           const uint32_t* pos_ctx, int n_ctx, uint32_t noise_start, int n_rows, bool causal, float* partials, uint32_t ctx_capacity,
                           int* err, int* n_records_out);
dfl_status launch_kv_tiled_to_rows(cudaStream_t st, const void* tiled, bool is_v, int n_kv, uint32_t pos0, uint32_t n_pos, void* rows);
dfl_status launch_kv_rows_to_tiled(cudaStream_t st, const void* rows, bool is_v, int n_kv, uint32_t pos0, uint32_t n_pos, void* tiled);
// tensor-core span kernel over an fp16 cache (attn_tc.cu)
bool attn_tc_supported(const AttnGeom& g, bool kv_f16);
int attn_tc_chunks_per_span(const AttnGeom& g, uint32_t kv_capacity);
// drafter attention on the tensor cores (f32 context cache split into f16 hi + lo on the way into shared memory)
bool dattn_tc_supported(const AttnGeom& g);
dfl_status launch_dattn_span_tc(cudaStream_t st, const AttnGeom& g, const float* q_rot, const float* k_ctx, const float* v_ctx,
                                const uint32_t* pos_ctx, int ctx_begin, int n_ctx, const float* k_noise, const float* v_noise,
                                uint32_t noise_start, int n_rows, bool causal, uint32_t window, float* partials, uint32_t ctx_capacity,
                                int* n_spans_out);
dfl_status launch_attn_span_tc(cudaStream_t st, const AttnGeom& g, const float* q_rot, const void* k_cache, const void* v_cache,
                               uint32_t start, int n_rows, float* partials, int chunks_per_span);
uint64_t attn_partials_floats(const AttnGeom& g, uint32_t max_positions);

// ---- gated delta net (gdn.cu) --------------------------------------------------
struct GdnGeom {
    int n_v, n_k, hd, conv_k;  // hd must be 128, conv_k 4
    __host__ __device__ int conv_dim() const { return (2 * n_k + n_v) * hd; }
};
// The conv + norm stage of one GDN layer (oracle: forward.rs:985-1050), as data: inputs are the split-K partial sums of
// the qkv projection.
struct GdnFrontParams {
    GdnGeom g{};
    const float* part = nullptr;   // [splits][16][ld_part], this projection's columns first
    int splits = 0, ld_part = 0, n_rows = 0;
    const float* conv_w = nullptr; // [conv_dim][4]
    float* conv_state = nullptr;   // [3][conv_dim], updated in place
    float* qkv_raw = nullptr;      // [16][conv_dim] rows of the block before the convolution (kept for rollback)
    float *q_n = nullptr, *k_n = nullptr, *v_out = nullptr;
    float* conv_pre = nullptr;     // [3][conv_dim] the conv state before the block (kept for rollback)
};
#ifdef __CUDACC__
// The three conv-state rows of head `head` (128 channels) that precede the block, for the lane's four channels.  Only
// the warp that owns rows 0..3 needs them; it reads them before any warp of the CTA starts to write the new state.
__device__ __forceinline__ void gdn_front_old_state(const GdnFrontParams& p, int head, int lane, float4 (&old)[3]) {
    const int c = head * 128 + 4 * lane, conv_dim = p.g.conv_dim();
#pragma unroll
    for (int t = 0; t < 3; ++t) old[t] = __ldcg(reinterpret_cast<const float4*>(p.conv_state + t * conv_dim + c));
}
// conv1d (4 taps) + SiLU over the block's rows and the L2 norm of q / k heads, for one head of 128 channels by four
// warps: warp w owns rows 4w .. 4w + 3, lane owns channels 4 lane .. 4 lane + 3, so that a row's norm is one warp
// reduction.  `old` = gdn_front_old_state (used by warp 0 only).  A row's result does not depend on n_rows.
__device__ __forceinline__ void gdn_front_tile(const GdnFrontParams& p, int head, int w, int lane, const float4 (&old)[3]) {
    const int conv_dim = p.g.conv_dim(), i0 = 4 * w, c = head * 128 + 4 * lane;
    // xv[k] = input at row i0 - 3 + k (rows before the block come from the conv state)
    float4 xv[7];
#pragma unroll
    for (int k = 0; k < 7; ++k) {
        const int row = i0 - 3 + k;
        xv[k] = (row < 0 && w == 0) ? old[k < 3 ? k : 0] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll 2
    for (int s = 0; s < p.splits; ++s) {
        const float* base = p.part + (uint64_t)s * MAX_ROWS * p.ld_part + c;
#pragma unroll
        for (int k = 0; k < 7; ++k) {
            const int row = i0 - 3 + k;
            if (row >= 0 && row < p.n_rows) {
                const float4 a = __ldcg(reinterpret_cast<const float4*>(base + (uint64_t)row * p.ld_part));
                xv[k].x += a.x; xv[k].y += a.y; xv[k].z += a.z; xv[k].w += a.w;
            }
        }
    }
    if (p.conv_pre && w == 0) {   // the pre-block rows a partial accept restores from
#pragma unroll
        for (int t = 0; t < 3; ++t) *reinterpret_cast<float4*>(p.conv_pre + t * conv_dim + c) = xv[t];
    }
    // filter taps of the lane's four channels
    float4 tap[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) tap[e] = *reinterpret_cast<const float4*>(p.conv_w + (uint64_t)(c + e) * 4);
    float y[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const bool live = i0 + j < p.n_rows;
        if (live) *reinterpret_cast<float4*>(p.qkv_raw + (uint64_t)(i0 + j) * conv_dim + c) = xv[j + 3];
        const float in[4][4] = {{xv[j].x, xv[j + 1].x, xv[j + 2].x, xv[j + 3].x}, {xv[j].y, xv[j + 1].y, xv[j + 2].y, xv[j + 3].y},
                                {xv[j].z, xv[j + 1].z, xv[j + 2].z, xv[j + 3].z}, {xv[j].w, xv[j + 1].w, xv[j + 2].w, xv[j + 3].w}};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            // s = sum_k w[k] * window[k], k ascending (forward.rs:1000-1010)
            float sacc = 0.f;
            sacc += tap[e].x * in[e][0];
            sacc += tap[e].y * in[e][1];
            sacc += tap[e].z * in[e][2];
            sacc += tap[e].w * in[e][3];
            y[j][e] = live ? silu_f(sacc) : 0.f;
        }
    }
    // new state = the last three rows of {old state rows, block rows}: row n_rows + t of that sequence, t = 0..2
#pragma unroll
    for (int t = 0; t < 3; ++t) {
        const int v = p.n_rows + t;          // index into the virtual sequence
        if (v < 3) {
            if (w == 0) *reinterpret_cast<float4*>(p.conv_state + t * conv_dim + c) = xv[v];
        } else if (v - 3 >= i0 && v - 3 < i0 + 4) {
            *reinterpret_cast<float4*>(p.conv_state + t * conv_dim + c) = xv[v - 3 - i0 + 3];
        }
    }
    const bool is_v = head >= 2 * p.g.n_k;
    if (!is_v) {
        // y / max(||y||, eps) over the head's 128 channels (forward.rs:1269-1275)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float sq = warp_sum((y[j][0] * y[j][0] + y[j][1] * y[j][1]) + (y[j][2] * y[j][2] + y[j][3] * y[j][3]));
            const float inv = 1.0f / fmaxf(sqrtf(sq), 1e-6f);
#pragma unroll
            for (int e = 0; e < 4; ++e) y[j][e] *= inv;
        }
    }
    float* dst = is_v ? p.v_out + (uint64_t)(head - 2 * p.g.n_k) * 128 + 4 * lane
                      : (head < p.g.n_k ? p.q_n + (uint64_t)head * 128 + 4 * lane : p.k_n + (uint64_t)(head - p.g.n_k) * 128 + 4 * lane);
    const int dst_ld = is_v ? p.g.n_v * 128 : p.g.n_k * 128;
#pragma unroll
    for (int j = 0; j < 4; ++j)
        if (i0 + j < p.n_rows) *reinterpret_cast<float4*>(dst + (uint64_t)(i0 + j) * dst_ld) = make_float4(y[j][0], y[j][1], y[j][2], y[j][3]);
}
#endif
// conv1d + SiLU over the block, q/k L2 norm; keeps raw qkv rows for rollback; updates conv state in place.
dfl_status launch_gdn_front_p(cudaStream_t st, const GdnFrontParams& p);
dfl_status launch_gdn_front(cudaStream_t st, const GdnGeom& g, const float* part_qkv, int splits, int ld_part, int n_rows,
                            const float* conv_w, float* conv_state, float* qkv_raw, float* q_n, float* k_n, float* v, float* conv_pre = nullptr);
// Sequential delta-rule scan over n_rows tokens from state_in to state_out (different buffers).  With `acts` it also
// applies y = rmsnorm(o; eps*hd) * w * silu(z), z = sum of the z-GEMM partials, and packs the activations of out_proj;
// acts == nullptr advances the state only (the re-scan of a partial accept).
dfl_status launch_gdn_scan(cudaStream_t st, const GdnGeom& g, const float* state_in, float* state_out, const float* q_n,
                           const float* k_n, const float* v, const float* ab, const float* dt_bias, const float* a_log,
                           int n_rows, const float* part_z, int z_splits, int ld_part, const float* norm_w, uint8_t* acts,
                           int act_layout, int* err);
// conv state := last (conv_k-1) rows of {pre-block conv rows, raw qkv rows 0..n_keep-1}
dfl_status launch_gdn_conv_restore(cudaStream_t st, const GdnGeom& g, const float* conv_pre, const float* qkv_raw, int n_keep,
                                   float* conv_state);

// ---- drafter attention (drafter_attn.cu) ---------------------------------------
dfl_status launch_drafter_attn(cudaStream_t st, const AttnGeom& g, const float* q_rot, const float* k_ctx, const float* v_ctx,
                               const int32_t* pos_ctx, int ctx_begin, int ctx_len, const float* k_noise, const float* v_noise,
                               uint32_t noise_start, int n_rows, bool causal, uint32_t window, float* partials, uint8_t* acts,
                               int act_layout, int* err, uint32_t ctx_capacity = 0);

// top-16 (id, value) per row, descending, total order with ties to the lower index (kernel_topk16_f32,
// kernels/dflash2.metal:96-170); ids / vals [n_rows][16]; scratch of topk16_scratch_bytes(n_rows)
uint64_t topk16_scratch_bytes(int n_rows);
dfl_status launch_topk16(cudaStream_t st, const float* x, int n_rows, uint64_t n, uint64_t ld, int32_t* ids, float* vals, void* scratch);

}  // namespace dfl
