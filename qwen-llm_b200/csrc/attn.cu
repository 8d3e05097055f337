// Gated full-attention block of the verify pass (oracle: Forward::attn_step,
// crates/qwen-llm/src/forward.rs:834-932; reference GPU path metal_dflash.rs:9823-10099,
// kernels/attn.metal:137-196,266-336, kernels/attn_v4.metal:65-265).
//
// Unlike the reference, which scans the KV cache once per query row, all query rows of the
// block and all query heads of a GQA group share ONE pass over each 64-position KV chunk
// (row r attends to positions <= start + r), with per-chunk partial softmax results combined
// afterwards.  Q stays f32; scores, exp and sums are f32 with accurate expf.
#include "ops.cuh"

namespace dfl {

// ---- front: reduce GEMM partials, per-head RMSNorm, partial NeoX RoPE, KV append ---------
// grid (heads = n_q + 2 n_kv, n_rows), block = 128 threads (4 warps cooperate on one head).
__global__ void __launch_bounds__(128) attn_front_kernel(AttnGeom g, int gated, const float* part, int splits,
                                                         int ld_part, const float* __restrict__ q_norm_w,
                                                         const float* __restrict__ k_norm_w, uint32_t start, void* k_cache,
                                                         void* v_cache, int kv_mode, float* q_rot,
                                                         float* gate, const uint32_t* pos_override, long long cache_row0) {
    pdl_prologue();
    extern __shared__ float sh[];  // [hd] values, then 4 partial sums
    const int head = blockIdx.x, tok = blockIdx.y, hd = g.hd;
    const int q_stride = gated ? 2 * hd : hd;
    const int q_cols = g.n_q * q_stride, kv_cols = g.n_kv * hd;
    int kind, h, col0;  // 0 = q, 1 = k, 2 = v
    if (head < g.n_q) { kind = 0; h = head; col0 = h * q_stride; }
    else if (head < g.n_q + g.n_kv) { kind = 1; h = head - g.n_q; col0 = q_cols + h * hd; }
    else { kind = 2; h = head - g.n_q - g.n_kv; col0 = q_cols + kv_cols + h * hd; }
    const uint32_t pos = pos_override ? pos_override[tok] : start + (uint32_t)tok;  // RoPE position
    const uint64_t crow = cache_row0 >= 0 ? (uint64_t)cache_row0 + tok : pos;         // cache row
    float ss = 0.f;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float v = 0.f, gt = 0.f;
        for (int s = 0; s < splits; ++s) {
            const float* row = part + ((uint64_t)s * MAX_ROWS + tok) * ld_part;
            v += row[col0 + d];
            if (kind == 0 && gated) gt += row[col0 + hd + d];
        }
        sh[d] = v;
        ss += v * v;
        if (kind == 0 && gated) gate[(uint64_t)tok * (g.n_q * hd) + h * hd + d] = gt;
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) sh[hd + (threadIdx.x >> 5)] = ss;
    __syncthreads();
    if (kind == 2) {
        for (int d = threadIdx.x; d < hd; d += blockDim.x) {
            const uint64_t o = (crow * g.n_kv + h) * hd + d;
            if (kv_mode == KV_F16_TILED)
                reinterpret_cast<__half*>(v_cache)[kv_tile_base((uint32_t)crow, g.n_kv, h) + kv_tile_v_off((uint32_t)crow % KV_TILE_KEYS, d)] = __float2half_rn(sh[d]);
            else if (kv_mode == KV_F16_ROWS) reinterpret_cast<__half*>(v_cache)[o] = __float2half_rn(sh[d]);
            else reinterpret_cast<float*>(v_cache)[o] = sh[d];
        }
        return;
    }
    const float total = sh[hd] + sh[hd + 1] + sh[hd + 2] + sh[hd + 3];
    const float scale = 1.0f / sqrtf(total / (float)hd + g.eps);
    const float* nw = kind == 0 ? q_norm_w : k_norm_w;
    __syncthreads();
    for (int d = threadIdx.x; d < hd; d += blockDim.x) sh[d] = sh[d] * scale * nw[d];
    __syncthreads();
    const int half = g.n_rot / 2;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float out = sh[d];
        if (d < g.n_rot) {
            const int i = d < half ? d : d - half;
            const float exponent = (float)(2 * i) / (float)g.n_rot;
            const float freq = (float)pos / powf(g.theta, exponent);
            float sn, cs;
            sincosf(freq, &sn, &cs);
            const float a = sh[i], b = sh[i + half];
            out = d < half ? (a * cs - b * sn) : (a * sn + b * cs);
        }
        if (kind == 0) q_rot[((uint64_t)tok * g.n_q + h) * hd + d] = out;
        else {
            const uint64_t o = (crow * g.n_kv + h) * hd + d;
            if (kv_mode == KV_F16_TILED)
                reinterpret_cast<__half*>(k_cache)[kv_tile_base((uint32_t)crow, g.n_kv, h) + kv_tile_k_off((uint32_t)crow % KV_TILE_KEYS, d)] = __float2half_rn(out);
            else if (kv_mode == KV_F16_ROWS) reinterpret_cast<__half*>(k_cache)[o] = __float2half_rn(out);
            else reinterpret_cast<float*>(k_cache)[o] = out;
        }
    }
}

dfl_status launch_attn_front(cudaStream_t st, const AttnGeom& g, bool gated, const float* part, int splits, int ld_part,
                             const float* q_norm_w, const float* k_norm_w, uint32_t start, int n_rows, void* k_cache,
                             void* v_cache, int kv_mode, float* q_rot, float* gate, const uint32_t* pos_override, long long cache_row0) {
    dim3 grid((unsigned)(g.n_q + 2 * g.n_kv), (unsigned)n_rows);
    launch_k(attn_front_kernel, dim3(grid), dim3(128), (g.hd + 4) * sizeof(float), st, g, gated ? 1 : 0, part, splits, ld_part, q_norm_w, k_norm_w, start,
                                                                   k_cache, v_cache, kv_mode, q_rot, gate, pos_override, cache_row0);
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

// ---- chunk kernel ----------------------------------------------------------------------
// grid (n_chunks, n_kv), block 256.  partial record per (chunk, kv head, query): [m, l, acc[hd]].
template <typename KV, int HD>
__global__ void __launch_bounds__(256) attn_chunk_kernel(AttnGeom g, const float* q_rot, const KV* k_cache,
                                                         const KV* v_cache, uint32_t start, int n_rows,
                                                         float* partials, int rows_per_cta) {
    pdl_prologue();
    extern __shared__ float sm[];
    constexpr int LD = HD + 1;
    float* ks = sm;                      // [64][LD]
    float* vs = ks + ATTN_CHUNK * LD;    // [64][LD]
    float* qs = vs + ATTN_CHUNK * LD;    // [8 warps][HD]
    float* ps = qs + 8 * HD;             // [8 warps][64]
    const int chunk = blockIdx.x, kvh = blockIdx.y;
    const int group = g.n_q / g.n_kv;
    const uint32_t n_pos = start + (uint32_t)n_rows;
    const uint32_t p0 = (uint32_t)chunk * ATTN_CHUNK;
    const int n_here = (int)min((uint32_t)ATTN_CHUNK, n_pos - p0);
    // 16-byte vector loads, all issued before the first use (one latency round per CTA)
    constexpr int EPV = 16 / (int)sizeof(KV);          // elements per vector
    constexpr int VPR = HD / EPV;                      // vectors per cache row
    constexpr int ITERS = ATTN_CHUNK * VPR / 256;
    uint4 kreg[ITERS], vreg[ITERS];
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        const int idx = threadIdx.x + it * 256, kp = idx / VPR, vv = idx % VPR;
        kreg[it] = make_uint4(0, 0, 0, 0);
        vreg[it] = make_uint4(0, 0, 0, 0);
        if (kp < n_here) {
            const uint64_t o = ((uint64_t)(p0 + kp) * g.n_kv + kvh) * HD + vv * EPV;
            kreg[it] = *reinterpret_cast<const uint4*>(k_cache + o);
            vreg[it] = *reinterpret_cast<const uint4*>(v_cache + o);
        }
    }
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        const int idx = threadIdx.x + it * 256, kp = idx / VPR, vv = idx % VPR;
        const KV* ke = reinterpret_cast<const KV*>(&kreg[it]);
        const KV* ve = reinterpret_cast<const KV*>(&vreg[it]);
#pragma unroll
        for (int e = 0; e < EPV; ++e) {
            ks[kp * LD + vv * EPV + e] = (float)ke[e];
            vs[kp * LD + vv * EPV + e] = (float)ve[e];
        }
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float scale = 1.0f / sqrtf((float)HD);
    // blockIdx.z selects a group of query rows: four per CTA at short context so that the GPU still fills, all sixteen
    // once there are enough KV chunks (every row group re-reads the chunk, which is what long contexts must avoid)
    const int q_lo = blockIdx.z * rows_per_cta * group;
    const int q_hi = min(n_rows, ((int)blockIdx.z + 1) * rows_per_cta) * group;
    float* myq = qs + warp * HD;
    float* myp = ps + warp * ATTN_CHUNK;
    for (int qi = q_lo + warp; qi < q_hi; qi += 8) {
        const int row = qi / group, qh = kvh * group + qi % group;
        const float* qsrc = q_rot + ((uint64_t)row * g.n_q + qh) * HD;
        for (int d = lane; d < HD; d += 32) myq[d] = qsrc[d];
        __syncwarp();
        const uint32_t last = start + (uint32_t)row;  // last visible position
        float s0 = 0.f, s1 = 0.f;
        const float* k0 = ks + lane * LD;
        const float* k1 = ks + (lane + 32) * LD;
#pragma unroll 8
        for (int d = 0; d < HD; ++d) {
            const float qv = myq[d];
            s0 = fmaf(qv, k0[d], s0);
            s1 = fmaf(qv, k1[d], s1);
        }
        s0 *= scale;
        s1 *= scale;
        const bool ok0 = lane < n_here && p0 + lane <= last;
        const bool ok1 = lane + 32 < n_here && p0 + lane + 32 <= last;
        if (!ok0) s0 = -INFINITY;
        if (!ok1) s1 = -INFINITY;
        const float m = warp_max(fmaxf(s0, s1));
        float e0 = 0.f, e1 = 0.f;
        if (m > -INFINITY) {
            e0 = ok0 ? expf(s0 - m) : 0.f;
            e1 = ok1 ? expf(s1 - m) : 0.f;
        }
        const float l = warp_sum(e0 + e1);
        myp[lane] = e0;
        myp[lane + 32] = e1;
        __syncwarp();
        float acc[HD / 32];
#pragma unroll
        for (int j = 0; j < HD / 32; ++j) acc[j] = 0.f;
        for (int kp = 0; kp < n_here; ++kp) {
            const float pw = myp[kp];
#pragma unroll
            for (int j = 0; j < HD / 32; ++j) acc[j] = fmaf(pw, vs[kp * LD + lane + 32 * j], acc[j]);
        }
        float* rec = partials + (((uint64_t)chunk * g.n_kv + kvh) * (MAX_ROWS * group) + qi) * (HD + 2);
        if (lane == 0) { rec[0] = m; rec[1] = l; }
#pragma unroll
        for (int j = 0; j < HD / 32; ++j) rec[2 + lane + 32 * j] = acc[j];
        __syncwarp();
    }
}

// ---- combine + sigmoid gate + activation packing ---------------------------------------------
// grid (n_q, n_rows), block 32: one warp per (row, q head); lane owns hd/32 consecutive dims.
template <int HD>
__global__ void __launch_bounds__(32) attn_post_kernel(AttnGeom g, const float* partials, int pos_per_span, int recs_per_span,
                                                       const float* gate, uint32_t start, uint8_t* acts, int bf3,
                                                       float* out_f32, int* err) {
    pdl_prologue();
    constexpr int PER = HD / 32;  // 4 or 8
    const int qh = blockIdx.x, row = blockIdx.y, lane = threadIdx.x;
    const int group = g.n_q / g.n_kv, kvh = qh / group, qi = row * group + qh % group;
    // records holding visible positions: one per 64-position chunk (scalar kernel), one per span of chunks (mma.sync
    // kernel) or two per span of tiles (tcgen05 kernel: one per half of the keys)
    const int n_chunks = ((int)((start + (uint32_t)row) / (uint32_t)pos_per_span) + 1) * recs_per_span;
    float M = -INFINITY;
    for (int c = lane; c < n_chunks; c += 32) {
        const float* rec = partials + (((uint64_t)c * g.n_kv + kvh) * (MAX_ROWS * group) + qi) * (HD + 2);
        M = fmaxf(M, rec[0]);
    }
    M = warp_max(M);
    float acc[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) acc[j] = 0.f;
    float L = 0.f;
    // records are merged in index order; their loads are issued eight records at a time so that the latency of one
    // round trip covers eight records (a long context has dozens)
    constexpr int BATCH = 8;
    const uint64_t rec_stride = (uint64_t)g.n_kv * (MAX_ROWS * group) * (HD + 2);
    const float* rec0 = partials + ((uint64_t)kvh * (MAX_ROWS * group) + qi) * (HD + 2);
    for (int c0 = 0; c0 < n_chunks; c0 += BATCH) {
        float mb[BATCH], lb[BATCH], vb[BATCH][PER];
#pragma unroll
        for (int u = 0; u < BATCH; ++u) {
            const int c = c0 + u < n_chunks ? c0 + u : n_chunks - 1;
            const float* rec = rec0 + (uint64_t)c * rec_stride;
            mb[u] = rec[0];
            lb[u] = rec[1];
#pragma unroll
            for (int j = 0; j < PER; ++j) vb[u][j] = rec[2 + lane * PER + j];
        }
#pragma unroll
        for (int u = 0; u < BATCH; ++u) {
            if (c0 + u >= n_chunks || mb[u] == -INFINITY) continue;
            const float f = expf(mb[u] - M);
            L = fmaf(lb[u], f, L);
#pragma unroll
            for (int j = 0; j < PER; ++j) acc[j] = fmaf(vb[u][j], f, acc[j]);
        }
    }
    const float inv = 1.0f / L;
    const int col0 = qh * HD + lane * PER;
    float v[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        v[j] = acc[j] * inv;
        if (gate) v[j] *= sigmoid_f(gate[(uint64_t)row * (g.n_q * HD) + col0 + j]);
    }
    if (out_f32)
#pragma unroll
        for (int j = 0; j < PER; ++j) out_f32[(uint64_t)row * (g.n_q * HD) + col0 + j] = v[j];
    if (acts) {
        bool over = false;
        float sum = 0.f;
#pragma unroll
        for (int q4 = 0; q4 < PER / 4; ++q4) {
            const int col = col0 + 4 * q4;
            uint8_t* chunk = acts + (uint64_t)(col >> 8) * act_chunk_dev(bf3);
            const float quad[4] = {v[4 * q4], v[4 * q4 + 1], v[4 * q4 + 2], v[4 * q4 + 3]};
            pack_quad_any(chunk, bf3, row, col & 255, quad, over);
            sum += quad[0] + quad[1] + quad[2] + quad[3];
        }
        if ((bf3 == ACT_F16 || bf3 == ACT_TS)) {
            // 32-column sub-block sums: 32 / PER lanes each
            constexpr int LANES = 32 / PER;
#pragma unroll
            for (int o = LANES / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            if ((lane % LANES) == 0) {
                uint8_t* chunk = acts + (uint64_t)(col0 >> 8) * act_chunk_dev(bf3);
                store_subsum(chunk, bf3, row, (col0 & 255) >> 5, sum, over);
            }
        }
        if (over) atomicCAS(err, 0, DEV_ERR_OVERFLOW);
    }
}

// zero the activation rows of padded tokens (rows n_rows..15) and the plane padding
__global__ void acts_clear_kernel(uint8_t* acts, uint64_t bytes) {
    pdl_prologue();
    const uint64_t i = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) * 16;
    if (i < bytes) *reinterpret_cast<uint4*>(acts + i) = make_uint4(0, 0, 0, 0);
}
dfl_status launch_acts_clear(cudaStream_t st, uint8_t* acts, uint64_t bytes) {
    launch_k(acts_clear_kernel, dim3((unsigned)((bytes / 16 + 255) / 256)), dim3(256), 0, st, acts, bytes);
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

uint64_t attn_partials_floats(const AttnGeom& g, uint32_t max_positions) {
    const uint64_t chunks = (max_positions + ATTN_CHUNK - 1) / ATTN_CHUNK;
    return chunks * g.n_kv * (uint64_t)(MAX_ROWS * (g.n_q / g.n_kv)) * (g.hd + 2);
}

template <typename KV, int HD>
static dfl_status launch_chunk(cudaStream_t st, const AttnGeom& g, const float* q_rot, const void* k_cache, const void* v_cache,
                               uint32_t start, int n_rows, float* partials, int n_chunks) {
    const size_t smem = (size_t)(2 * ATTN_CHUNK * (HD + 1) + 8 * HD + 8 * ATTN_CHUNK) * sizeof(float);
    static bool set = false;
    if (!set) {
        DFL_CUDA(cudaFuncSetAttribute(attn_chunk_kernel<KV, HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        set = true;
    }
    int rows_per_cta = (long long)n_chunks * g.n_kv >= 2 * sm_count() ? MAX_ROWS : ATTN_ROW_GROUP;
    // Short contexts leave most SMs idle at four rows per CTA: narrow the row group while every warp still has a query.
    const int group = g.n_q / g.n_kv;
    while (rows_per_cta > 1 && rows_per_cta <= ATTN_ROW_GROUP && (rows_per_cta / 2) * group >= 8 &&
           (long long)n_chunks * g.n_kv * ((n_rows + rows_per_cta - 1) / rows_per_cta) < sm_count())
        rows_per_cta /= 2;
    if (const char* e = getenv("DFL_ATTN_ROWS_PER_CTA")) {   // test hook: results must not depend on the grouping
        const int v = atoi(e);
        if (v == 1 || v == 2 || v == 4 || v == 8 || v == 16) rows_per_cta = v;
    }
    launch_k(attn_chunk_kernel<KV, HD>, dim3((unsigned)n_chunks, (unsigned)g.n_kv, (unsigned)((n_rows + rows_per_cta - 1) / rows_per_cta)), dim3(256), smem, st,
              g, q_rot, reinterpret_cast<const KV*>(k_cache), reinterpret_cast<const KV*>(v_cache), start, n_rows, partials, rows_per_cta);
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

dfl_status launch_attn_verify(cudaStream_t st, const AttnGeom& g, const float* q_rot, const float* gate, const void* k_cache,
                              const void* v_cache, int kv_mode, uint32_t start, int n_rows, float* partials, uint8_t* acts, int bf3,
                              float* out_f32, int* err, uint32_t kv_capacity) {
    if (g.hd != 128 && g.hd != 256) return fail(DFL_ERR_UNSUPPORTED, "attention: head_dim must be 128 or 256");
    const int n_chunks = (int)((start + (uint32_t)n_rows + ATTN_CHUNK - 1) / ATTN_CHUNK);
    dfl_status s;
    const bool kv_f16 = kv_mode != KV_F32_ROWS;
    int pos_per_span = ATTN_CHUNK, recs_per_span = 1;
    const char* tc_env = getenv("DFL_ATTN_TC");
    if (kv_mode == KV_F16_TILED) {
        const int cps = attn_t5_chunks_per_span(g, kv_capacity);
        pos_per_span = cps * KV_TILE_KEYS;
        recs_per_span = 2;
        s = launch_attn_t5(st, g, q_rot, k_cache, v_cache, start, n_rows, partials, cps, err);
    } else if (attn_tc_supported(g, kv_f16) && !(tc_env && tc_env[0] == '0')) {
        const int cps = attn_tc_chunks_per_span(g, kv_capacity);
        pos_per_span = cps * ATTN_CHUNK;
        s = launch_attn_span_tc(st, g, q_rot, k_cache, v_cache, start, n_rows, partials, cps);
    } else if (g.hd == 128) s = kv_f16 ? launch_chunk<__half, 128>(st, g, q_rot, k_cache, v_cache, start, n_rows, partials, n_chunks)
                                : launch_chunk<float, 128>(st, g, q_rot, k_cache, v_cache, start, n_rows, partials, n_chunks);
    else s = kv_f16 ? launch_chunk<__half, 256>(st, g, q_rot, k_cache, v_cache, start, n_rows, partials, n_chunks)
                    : launch_chunk<float, 256>(st, g, q_rot, k_cache, v_cache, start, n_rows, partials, n_chunks);
    DFL_CHECK(s);
    if (acts && n_rows < MAX_ROWS) {
        // rows of absent tokens must read as zero in the next GEMM
        DFL_CHECK(launch_acts_clear(st, acts, (uint64_t)g.n_q * g.hd / TILE_K * (uint64_t)act_chunk_bytes(bf3)));
    }
    (void)n_chunks;
    if (g.hd == 128) launch_k(attn_post_kernel<128>, dim3(dim3((unsigned)g.n_q, (unsigned)n_rows)), dim3(32), 0, st, g, partials, pos_per_span, recs_per_span, gate, start, acts, bf3, out_f32, err);
    else launch_k(attn_post_kernel<256>, dim3(dim3((unsigned)g.n_q, (unsigned)n_rows)), dim3(32), 0, st, g, partials, pos_per_span, recs_per_span, gate, start, acts, bf3, out_f32, err);
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

}  // namespace dfl
