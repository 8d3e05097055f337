// Few-row weight-streaming GEMM on the fifth-generation tensor cores.
//
// Same contract as the mma.sync kernel (gemm_fewrow.cu: y[r, o] = sum_i x[r, i] W[o, i], <= 16
// activation rows, split-K partials, deterministic), different engine.  One CTA per SM, four
// kinds of warps that only meet at mbarriers:
//   * a producer thread streams 128-row x 256-column stages of packed weights with bulk copies
//     into a shared-memory ring; the packed activations of the CTA's column range are copied
//     once and stay resident as the B operand;
//   * sixteen unpacking warps turn the integer quants into exact f16 integers q * sc (the
//     6-bit sub-block scale folded in, still exact: q * sc < 2048) and store them with
//     tcgen05.st into tensor memory, thread = (row, quarter of the columns), row = TMEM lane.
//     They do nothing else, so their instruction stream never waits for an accumulator;
//   * four warps, one per scheduler, issue tcgen05.mma (A from tensor memory, B = activations
//     hi / lo planes from shared memory, M = 128, N = 32, K = 16 per instruction), sixteen per
//     256-column block, accumulating it in tensor memory; a seventeenth MMA multiplies the
//     sub-block mins with the per-sub-block activation sums (the K-quant "min" term);
//   * four draining warps (thread = weight row) read the finished block's accumulator back
//     (tcgen05.ld), apply the per-row f16 super-block scales d and dmin in f32 and add to
//     sixteen register accumulators (one per token); at the end of a row tile they write the
//     partial result straight to global memory.  No shared-memory reduction, no atomics.
// The A operand and the accumulators are double-buffered in tensor memory: unpacking pass
// i + 1 overlaps the MMAs of pass i, which overlap the read-back of block i - 1.
#include <mutex>

#include "ops.cuh"
#include "tcgen05_prims.cuh"

namespace dfl {

// Q6_K packing lives in gemm_ts_q6k.cuh (included further down, after the primitives it uses)
__device__ __forceinline__ uint64_t src_block_index(uint64_t row, int kb, int kblocks, uint64_t n_out, int kb_group);
__global__ void retile_ts_q6k_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, uint64_t n_out, int kblocks, int kb_group);
__device__ float decode_ts_q6k_elem(const uint8_t* stage, int r, int k);
__global__ void retile_ts_q80_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, uint64_t n_out, int kblocks, int kb_group);
__device__ float decode_ts_q80_elem(const uint8_t* stage, int r, int k);
__global__ void q80_scale_range_kernel(const uint8_t* __restrict__ src, uint64_t n_blocks, int* flag);
__global__ void retile_tsb_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, uint64_t n_in, uint64_t n_out, int kblocks);
__device__ float decode_tsb_elem(const uint8_t* stage, int r, int k);

// ---------------------------------------------------------------------------------------------
// Re-tiling into row-lane tiles and the inverse decode.
// ---------------------------------------------------------------------------------------------
// Index of the ggml block (row, kb) in the source.  kb_group = 0: plain row-major [n_out][kblocks].  kb_group > 0: the
// source is [kblocks / kb_group] matrices of [n_out][kb_group] blocks one after the other (the experts of
// ffn_down_exps), viewed as one matrix whose columns are the experts' columns side by side.
__device__ __forceinline__ uint64_t src_block_index(uint64_t row, int kb, int kblocks, uint64_t n_out, int kb_group) {
    if (kb_group <= 0) return row * kblocks + kb;
    return ((uint64_t)(kb / kb_group) * n_out + row) * kb_group + kb % kb_group;
}

template <int DT>
__global__ void retile_ts_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, uint64_t n_out, int kblocks, int kb_group) {
    constexpr int SRC_BLK = DT == DFL_Q4_K ? 144 : DT == DFL_Q5_K ? 176 : 210;
    constexpr int STAGE = DT == DFL_Q4_K ? STAGE_Q4_K : DT == DFL_Q5_K ? STAGE_Q5_K : STAGE_Q6_K;
    const uint64_t tile_id = blockIdx.x;
    const int kb = (int)(tile_id % kblocks);
    const uint64_t rt = tile_id / kblocks;
    uint8_t* stage = dst + tile_id * STAGE;
    // one item = 16 destination bytes
    for (int idx = threadIdx.x; idx < STAGE / 16; idx += blockDim.x) {
        uint8_t out[16];
#pragma unroll
        for (int b = 0; b < 16; ++b) out[b] = 0;
        const int off = idx * 16;
        if (DT == DFL_Q4_K || DT == DFL_Q5_K) {
            const int qs_src = DT == DFL_Q4_K ? 16 : 48;
            int r, src_off;
            if (off < TSQ4_OFF_QS) { r = idx; src_off = 0; }                                  // header
            else if (off < TSQ4_OFF_QS + 16384) {                                             // qs [kp][half][row]
                const int i = idx - TSQ4_OFF_QS / 16;
                r = i & 127;
                src_off = qs_src + 32 * (i >> 8) + 16 * ((i >> 7) & 1);
            } else {                                                                          // Q5_K qh [half][row]
                const int i = idx - TSQ5_OFF_QH / 16;
                r = i & 127;
                src_off = 16 + 16 * (i >> 7);
            }
            const uint64_t row = rt * TILE_R + r;
            if (row < n_out) {
                const uint8_t* blk = src + src_block_index(row, kb, kblocks, n_out, kb_group) * (uint64_t)SRC_BLK + src_off;
#pragma unroll
                for (int b = 0; b < 16; ++b) out[b] = blk[b];
                if (off < TSQ4_OFF_QS) {
                    // header: d, dmin, then the eight (scale, min) pairs as 12-bit fields, pair j at bit 12 j
                    uint32_t f[3] = {0, 0, 0};
                    for (int j = 0; j < 8; ++j) {
                        uint32_t sc, m;
                        k4_scale_min(blk + 4, j, sc, m);
                        const uint64_t v = (uint64_t)(sc | (m << 6)) << ((12 * j) & 31);
                        f[(12 * j) >> 5] |= (uint32_t)v;
                        if (((12 * j) >> 5) < 2) f[((12 * j) >> 5) + 1] |= (uint32_t)(v >> 32);
                    }
                    for (int b = 0; b < 12; ++b) out[4 + b] = (uint8_t)(f[b >> 2] >> (8 * (b & 3)));
                }
            }
        }
        *reinterpret_cast<uint4*>(stage + off) = *reinterpret_cast<const uint4*>(out);
    }
}

dfl_status retile_matrix_ts(cudaStream_t st, int dtype, const uint8_t* ggml_dev, uint64_t n_in, uint64_t n_out, uint8_t* dst_tiles,
                            int kb_group) {
    if (n_in % TILE_K) return fail(DFL_ERR_BAD_SHAPE, "retile: n_in must be a multiple of 256");
    const int kblocks = (int)(n_in / TILE_K);
    const uint64_t n_tiles = (uint64_t)kblocks * ((n_out + TILE_R - 1) / TILE_R);
    if (n_tiles == 0 || n_tiles > 0x7fffffffu) return fail(DFL_ERR_BAD_SHAPE, "retile: tile count out of range");
    dim3 grid((unsigned)n_tiles), block(256);
    switch (dtype) {
        case DFL_Q4_K: retile_ts_kernel<DFL_Q4_K><<<grid, block, 0, st>>>(ggml_dev, dst_tiles, n_out, kblocks, kb_group); break;
        case DFL_Q5_K: retile_ts_kernel<DFL_Q5_K><<<grid, block, 0, st>>>(ggml_dev, dst_tiles, n_out, kblocks, kb_group); break;
        case DFL_Q6_K: retile_ts_q6k_kernel<<<grid, block, 0, st>>>(ggml_dev, dst_tiles, n_out, kblocks, kb_group); break;
        case DFL_Q8_0: retile_ts_q80_kernel<<<grid, block, 0, st>>>(ggml_dev, dst_tiles, n_out, kblocks, kb_group); break;
        case DFL_BF16:
            if (kb_group > 0) return fail(DFL_ERR_UNSUPPORTED, "retile: grouped column blocks are not built for bf16");
            retile_tsb_kernel<<<grid, block, 0, st>>>(ggml_dev, dst_tiles, n_in, n_out, kblocks);
            break;
        default: return fail(DFL_ERR_UNSUPPORTED, "retile: dtype has no row-lane tile layout");
    }
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

__global__ void decode_tiles_ts_kernel(const uint8_t* __restrict__ tiles, int dtype, uint64_t n_in, uint64_t n_out, int kblocks,
                                       float* __restrict__ out) {
    const uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_in * n_out) return;
    const uint64_t row = idx / n_in;
    const int kk = (int)(idx % n_in);
    const int kb = kk >> 8, k = kk & 255;
    const uint64_t rt = row / TILE_R;
    const int r = (int)(row % TILE_R);
    const uint8_t* stage = tiles + (rt * kblocks + kb) * (uint64_t)stage_bytes_of(dtype, LAYOUT_TS);
    float v = 0.f;
    if (dtype == DFL_Q4_K || dtype == DFL_Q5_K) {
        const uint8_t* h = stage + r * 16;
        const float d = __half2float(__ushort_as_half((unsigned short)(h[0] | (h[1] << 8))));
        const float dmin = __half2float(__ushort_as_half((unsigned short)(h[2] | (h[3] << 8))));
        const uint32_t* f = reinterpret_cast<const uint32_t*>(h + 4);
        const int bit = 12 * (k >> 5);
        const uint64_t two = (uint64_t)f[bit >> 5] | ((uint64_t)((bit >> 5) < 2 ? f[(bit >> 5) + 1] : 0u) << 32);
        const uint32_t pair = (uint32_t)(two >> (bit & 31)) & 0xfffu, sc = pair & 63u, m = pair >> 6;
        const int kp = k >> 6, hi = (k >> 5) & 1, l = k & 31;
        const uint8_t byte = stage[TSQ4_OFF_QS + ((kp * 2 + (l >> 4)) * 128 + r) * 16 + (l & 15)];
        uint32_t q = hi ? (byte >> 4) : (byte & 15);
        if (dtype == DFL_Q5_K) q |= ((stage[TSQ5_OFF_QH + ((l >> 4) * 128 + r) * 16 + (l & 15)] >> (2 * kp + hi)) & 1u) << 4;
        v = __fsub_rn(__fmul_rn(d * (float)sc, (float)q), dmin * (float)m);
    } else if (dtype == DFL_Q6_K) {
        v = decode_ts_q6k_elem(stage, r, k);
    } else if (dtype == DFL_Q8_0) {
        v = decode_ts_q80_elem(stage, r, k);
    } else if (dtype == DFL_BF16) {
        v = decode_tsb_elem(stage, r, k);
    }
    out[idx] = v;
}

// Whether every block scale of a Q8_0 matrix (ggml bytes on the device) leaves q * d inside the f16 range.
dfl_status q80_scales_fit_ts(cudaStream_t st, const uint8_t* ggml_dev, uint64_t n_in, uint64_t n_out, bool* fits) {
    int* flag = nullptr;
    DFL_CUDA(cudaMalloc(&flag, sizeof(int)));
    cudaMemsetAsync(flag, 0, sizeof(int), st);
    const uint64_t n_blocks = n_in / 32 * n_out;
    q80_scale_range_kernel<<<(unsigned)((n_blocks + 255) / 256), 256, 0, st>>>(ggml_dev, n_blocks, flag);
    count_launch();
    int h = 1;
    cudaError_t e = cudaMemcpyAsync(&h, flag, sizeof(int), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    cudaFree(flag);
    if (e != cudaSuccess) return fail(DFL_ERR_CUDA, std::string("q80 scale range: ") + cudaGetErrorString(e));
    *fits = h == 0;
    return DFL_OK;
}

dfl_status decode_tiles_ts(cudaStream_t st, const QMatrix& m, float* out_dev) {
    const uint64_t n = m.n_in * m.n_out;
    decode_tiles_ts_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(m.tiles, m.dtype, m.n_in, m.n_out, m.kblocks, out_dev);
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

// ---------------------------------------------------------------------------------------------
// Standalone activation packing (the model path packs inside its glue kernels).
// One CTA per 256-column block; thread = (token = tid / 16, 16 consecutive columns).
// ---------------------------------------------------------------------------------------------
__global__ void prep_acts_ts_kernel(const float* __restrict__ x, int ld, int n_rows, float pre_scale, uint8_t* __restrict__ acts,
                                    int* err) {
    const int kb = blockIdx.x, tok = threadIdx.x >> 4, seg = threadIdx.x & 15;
    uint8_t* chunk = acts + (uint64_t)kb * ACTTS_CHUNK;
    // the zero half of the small operand (sub-block index 8..15)
    for (int i = threadIdx.x; i < 768 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(chunk + TS_BMIN_OFF + 768)[i] = 0u;
    float v[16];
    if (tok < n_rows) {
        const float4* src = reinterpret_cast<const float4*>(x + (uint64_t)tok * ld + (uint64_t)kb * TILE_K + seg * 16);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float4 q = src[j];
            v[4 * j] = q.x * pre_scale; v[4 * j + 1] = q.y * pre_scale; v[4 * j + 2] = q.z * pre_scale; v[4 * j + 3] = q.w * pre_scale;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = 0.f;
    }
    bool over = false;
    float sum = 0.f;
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) {
        const float quad[4] = {v[4 * q4], v[4 * q4 + 1], v[4 * q4 + 2], v[4 * q4 + 3]};
        pack_quad_ts(chunk, tok, seg * 16 + 4 * q4, quad, over);
        sum += (quad[0] + quad[1]) + (quad[2] + quad[3]);
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);  // 32-column sub-block = this thread and its neighbour
    if ((seg & 1) == 0) pack_subsum_ts(chunk, tok, seg >> 1, sum, over);
    if (over) atomicCAS(err, 0, DEV_ERR_OVERFLOW);
}

dfl_status launch_prep_acts_ts(cudaStream_t st, const float* x, int ld, int n_rows, uint64_t k, float pre_scale, uint8_t* acts,
                               int* dev_err) {
    if (k % TILE_K || n_rows < 0 || n_rows > MAX_ROWS) return fail(DFL_ERR_BAD_SHAPE, "prep_acts: shape");
    prep_acts_ts_kernel<<<(unsigned)(k / TILE_K), 256, 0, st>>>(x, ld, n_rows, pre_scale, acts, dev_err);
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

// ---------------------------------------------------------------------------------------------
// tcgen05 / tensor-memory primitives (sm_100a).
// ---------------------------------------------------------------------------------------------
namespace ts {

constexpr int GROUP_WARPS = 8;                          // unpacking warps per group; thread = (row = 32 * (warp % 4) + lane, kp2 = (warp / 4) % 2)
constexpr int UNPACK_WARPS = 2 * GROUP_WARPS;           // two groups that take the entries alternately, so that their phases interleave
constexpr int DRAIN_WARP0 = 16, DRAIN_WARPS = 4;        // thread = weight row; warp % 4 = its quarter of the tensor-memory lanes
constexpr int MMA_WARP0 = 20, MMA_WARPS = 4;            // warp 20 + 2 g + c issues the MMAs of group g's halves h with h % 2 == c
constexpr int PRODUCER_WARP = 24;
constexpr int THREADS = 25 * 32;                        // 800
#ifndef DFL_TS_KC
#define DFL_TS_KC 6
#endif
constexpr int KC = DFL_TS_KC;                           // column blocks whose activations stay resident

// tensor-memory columns (32-bit each, 128 lanes), everything once per group: a 128-column A buffer (256 f16 per row)
// written and consumed in two halves, two 32-column accumulators (even / odd MMA steps), the 8-column A operand of the
// min term and its 48-column accumulator
constexpr uint32_t TM_A = 0, TM_A_STRIDE = 128, TM_D = 256, TM_D_STRIDE = 64, TM_AM = 384, TM_AM_STRIDE = 8, TM_DM = 400, TM_DM_STRIDE = 48,
                   TM_COLS = 512;
static_assert(TM_DM + 2 * TM_DM_STRIDE <= TM_COLS, "tensor memory budget");

__device__ __forceinline__ uint32_t h2sub(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("sub.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t h2mul(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t h2fma(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}
constexpr uint32_t MAGIC = 0x64006400u;      // half2(1024, 1024): 1024 + small integer in the mantissa
constexpr uint32_t H2_NEG1024 = 0xe400e400u; // half2(-1024)
constexpr uint32_t H2_16TH = 0x2c002c00u;    // half2(1/16)
constexpr uint32_t H2_NEG64 = 0xd400d400u;   // half2(-64)
// (a, b) small non-negative integers -> half2(a, b), exact
__device__ __forceinline__ uint32_t int_pair_h2(uint32_t a, uint32_t b) { return h2sub((a | (b << 16)) | MAGIC, MAGIC); }

struct UnitScales {
    float d, dmin;
};

template <int DT>
struct Fmt;

// Q4_K / Q5_K: two halves per stage.  In half h thread (row, kp2) takes the 64 columns of quarter kp = 2h + kp2:
// sub-blocks 2kp (low nibbles) and 2kp + 1 (high nibbles) of its row into r[0..15] / r[16..31]; r[c] = half2 of
// k-positions 2c, 2c + 1.
template <int DT>
struct FmtK45 {
    static constexpr int STAGE = DT == DFL_Q4_K ? STAGE_Q4_K : STAGE_Q5_K;
    static constexpr int STAGES = KC == 4 ? (DT == DFL_Q4_K ? 7 : 6) : (DT == DFL_Q4_K ? 6 : 5);
    static constexpr int HALVES = 2;
    static constexpr bool HAS_MIN = true;
    // MMA step jj (0..7) of half h multiplies A-buffer columns a_col .. + 8 with 16-column slice b_slice of the block
    __device__ static __forceinline__ uint32_t a_col(int h, int jj) { return (uint32_t)(64 * h + 8 * jj); }
    __device__ static __forceinline__ uint32_t b_slice(int h, int jj) { return (uint32_t)(8 * h + jj); }
    __device__ static __forceinline__ void store(uint32_t buf, int h, int kp2, const uint32_t (&r)[32]) { tmem_st32(buf + 64 * h + 32 * kp2, r); }
    __device__ static __forceinline__ int min_col(int h, int kp2) { return 2 * h + kp2; }
    __device__ static __forceinline__ void unpack(const uint8_t* st, int ps, int row, int kp2, uint32_t (&r)[32], uint32_t (&am)[8],
                                                  UnitScales& us) {
        const int kp = 2 * ps + kp2;
        const uint4 h = reinterpret_cast<const uint4*>(st)[row];
        const uint4* qs = reinterpret_cast<const uint4*>(st + TSQ4_OFF_QS);
        const uint4 qa = qs[(kp * 2 + 0) * 128 + row], qb = qs[(kp * 2 + 1) * 128 + row];
        us.d = __half2float(__ushort_as_half((unsigned short)(h.x & 0xffffu)));
        us.dmin = __half2float(__ushort_as_half((unsigned short)(h.x >> 16)));
        // (scale, min) pairs of sub-blocks 2kp and 2kp + 1: 24 bits at bit 24 kp of the 96-bit field h.y, h.z, h.w
        const uint32_t t = (ps == 0 ? (kp2 ? __funnelshift_r(h.y, h.z, 24) : h.y) : (kp2 ? (h.w >> 8) : __funnelshift_r(h.z, h.w, 16)));
        const uint32_t sc0 = t & 63u, m0 = (t >> 6) & 63u, sc1 = (t >> 12) & 63u, m1 = (t >> 18) & 63u;
        const uint32_t s0 = int_pair_h2(sc0, sc0), s1 = int_pair_h2(sc1, sc1);
        const uint32_t cml = s0, cal = h2mul(s0, H2_NEG1024);                      // (1024 + q) * sc - 1024 sc
        const uint32_t cmh = h2mul(s1, H2_16TH), cah = h2mul(s1, H2_NEG64);        // (1024 + 16 q) * sc / 16 - 64 sc
        const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
        if (DT == DFL_Q4_K) {
#pragma unroll
            for (int wi = 0; wi < 8; ++wi) {
                const uint32_t v = w[wi], v8 = v >> 8;
                r[2 * wi] = h2fma((v & 0x000f000fu) | MAGIC, cml, cal);
                r[2 * wi + 1] = h2fma((v8 & 0x000f000fu) | MAGIC, cml, cal);
                r[16 + 2 * wi] = h2fma((v & 0x00f000f0u) | MAGIC, cmh, cah);
                r[16 + 2 * wi + 1] = h2fma((v8 & 0x00f000f0u) | MAGIC, cmh, cah);
            }
        } else {
            const uint4* qh = reinterpret_cast<const uint4*>(st + TSQ5_OFF_QH);
            const uint4 ha = qh[row], hb = qh[128 + row];
            const uint32_t hw[8] = {ha.x, ha.y, ha.z, ha.w, hb.x, hb.y, hb.z, hb.w};
#pragma unroll
            for (int wi = 0; wi < 8; ++wi) {
                const uint32_t v = w[wi], v8 = v >> 8, t = hw[wi] >> (2 * kp);
                r[2 * wi] = h2fma((v & 0x000f000fu) | ((t << 4) & 0x00100010u) | MAGIC, cml, cal);
                r[2 * wi + 1] = h2fma((v8 & 0x000f000fu) | ((t >> 4) & 0x00100010u) | MAGIC, cml, cal);
                r[16 + 2 * wi] = h2fma((v & 0x00f000f0u) | ((t << 7) & 0x01000100u) | MAGIC, cmh, cah);
                r[16 + 2 * wi + 1] = h2fma((v8 & 0x00f000f0u) | ((t >> 1) & 0x01000100u) | MAGIC, cmh, cah);
            }
        }
        // column kp of the min-term A operand: the mins of this thread's two sub-blocks
        am[0] = int_pair_h2(m0, m1);
    }
};
template <>
struct Fmt<DFL_Q4_K> : FmtK45<DFL_Q4_K> {};
template <>
struct Fmt<DFL_Q5_K> : FmtK45<DFL_Q5_K> {};

}  // namespace ts

}  // namespace dfl

#include "gemm_ts_q6k.cuh"
#include "gemm_ts_q80.cuh"
#include "gemm_tsb.cuh"
#include "gemm_ts_kernel.cuh"
