// Verify attention over an fp16 KV cache on the tensor cores, for the long-context shape of the step
// (reference: kernel_attn_decode_* / attn_v4, kernels/attn_v4.metal:65-265; CPU oracle forward.rs:896-921).
//
// One CTA = one KV head x one span of `chunks_per_span` 64-position chunks; all 16 block rows x the 4 query
// heads of the GQA group (64 queries) share every K/V byte the CTA reads.  Per chunk:
//   S = Q K^T   mma.sync m16n8k16, Q (pre-scaled by 1/sqrt(hd)) as an exact f16 hi + lo pair, K straight from the cache
//   online softmax per query over the span (running max / sum in shared memory, f32)
//   O = O * alpha + P V   P as f16 hi + lo, V through ldmatrix.trans
// and one [m, l, O[128]] record per (span, query) at the end, merged by attn_post_kernel exactly like the per-chunk
// records of the scalar kernel.  Span boundaries are multiples of chunks_per_span * 64 positions and
// chunks_per_span depends only on the session's KV capacity, so a row's result does not depend on how many rows
// the call has or where the block starts (packed rows stay bitwise equal to single-token steps).
#include <cuda_fp16.h>

#include "ops.cuh"

namespace dfl {

namespace {
constexpr int TC_HD = 128, TC_GROUP = 4, TC_Q = MAX_ROWS * TC_GROUP;   // 64 queries per CTA
constexpr int TC_PITCH = 136;   // halfs per Q / K / V row in shared memory (272 B: conflict-free fragment loads)
constexpr int TC_PP = 72;       // halfs per P row
constexpr int TC_SP = 68;       // floats per S row
constexpr int TC_SMEM = (2 * TC_Q * TC_PITCH + 2 * ATTN_CHUNK * TC_PITCH + 2 * TC_Q * TC_PP) * 2 + TC_Q * TC_SP * 4 + 3 * TC_Q * 4;

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(smem_row)));
}
__device__ __forceinline__ uint32_t lds32(const __half* p) { return *reinterpret_cast<const uint32_t*>(p); }
}  // namespace

__global__ void __launch_bounds__(256) attn_span_tc_kernel(AttnGeom g, const float* q_rot, const __half* k_cache, const __half* v_cache,
                                                           uint32_t start, int n_rows, float* partials, int chunks_per_span) {
    pdl_prologue();
    extern __shared__ __align__(16) uint8_t sm_raw[];
    __half* q_hi = reinterpret_cast<__half*>(sm_raw);           // [64][136]
    __half* q_lo = q_hi + TC_Q * TC_PITCH;
    __half* ks = q_lo + TC_Q * TC_PITCH;                        // [64][136]
    __half* vs = ks + ATTN_CHUNK * TC_PITCH;
    __half* p_hi = vs + ATTN_CHUNK * TC_PITCH;                  // [64][72]
    __half* p_lo = p_hi + TC_Q * TC_PP;
    float* sf = reinterpret_cast<float*>(p_lo + TC_Q * TC_PP);  // [64][68]
    float* m_run = sf + TC_Q * TC_SP;                           // [64] running max, sum, last rescale factor
    float* l_run = m_run + TC_Q;
    float* alpha = l_run + TC_Q;

    const int span = blockIdx.x, kvh = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, t = lane & 3;
    const uint32_t n_pos = start + (uint32_t)n_rows;
    const float scale = 1.0f / sqrtf((float)TC_HD);

    // queries: pair = row * 4 + head-in-group, pre-scaled, split into exact f16 hi + lo
    for (int idx = threadIdx.x; idx < TC_Q * (TC_HD / 4); idx += 256) {
        const int pair = idx / (TC_HD / 4), d4 = (idx % (TC_HD / 4)) * 4;
        const int row = pair / TC_GROUP, qh = kvh * TC_GROUP + pair % TC_GROUP;
        float4 q = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row < n_rows) q = *reinterpret_cast<const float4*>(q_rot + ((uint64_t)row * g.n_q + qh) * TC_HD + d4);
        const float v[4] = {q.x * scale, q.y * scale, q.z * scale, q.w * scale};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const __half h = __float2half_rn(v[e]);
            q_hi[pair * TC_PITCH + d4 + e] = h;
            q_lo[pair * TC_PITCH + d4 + e] = __float2half_rn(v[e] - __half2float(h));
        }
    }
    if (threadIdx.x < TC_Q) { m_run[threadIdx.x] = -INFINITY; l_run[threadIdx.x] = 0.f; alpha[threadIdx.x] = 1.f; }

    const int mt = warp & 3, nh = warp >> 2;   // m-tile of 16 queries; half of the keys (S) / of the head dims (O)
    float o[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][j] = 0.f;

    const int c_begin = span * chunks_per_span;
    for (int c = c_begin; c < c_begin + chunks_per_span; ++c) {
        const uint32_t p0 = (uint32_t)c * ATTN_CHUNK;
        if (p0 >= n_pos) break;
        __syncthreads();   // previous chunk fully consumed (and the query planes written)
        // K / V rows of this chunk and head: 64 x 256 B each, 16 B per thread and step
        for (int idx = threadIdx.x; idx < ATTN_CHUNK * 16; idx += 256) {
            const int kp = idx >> 4, v16 = idx & 15;
            uint4 kk = make_uint4(0, 0, 0, 0), vv = make_uint4(0, 0, 0, 0);
            if (p0 + kp < n_pos) {
                const uint64_t off = ((uint64_t)(p0 + kp) * g.n_kv + kvh) * TC_HD + v16 * 8;
                kk = *reinterpret_cast<const uint4*>(k_cache + off);
                vv = *reinterpret_cast<const uint4*>(v_cache + off);
            }
            *reinterpret_cast<uint4*>(ks + kp * TC_PITCH + v16 * 8) = kk;
            *reinterpret_cast<uint4*>(vs + kp * TC_PITCH + v16 * 8) = vv;
        }
        __syncthreads();
        // ---- S = Q K^T for queries 16 mt .. +15, keys 32 nh .. +31 ----
        {
            float s[4][4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
            const __half* qa = q_hi + (16 * mt + gq) * TC_PITCH + 2 * t;
            const __half* qb = q_lo + (16 * mt + gq) * TC_PITCH + 2 * t;
#pragma unroll
            for (int kk = 0; kk < TC_HD / 16; ++kk) {
                const uint32_t h0 = lds32(qa + 16 * kk), h1 = lds32(qa + 8 * TC_PITCH + 16 * kk), h2 = lds32(qa + 16 * kk + 8),
                               h3 = lds32(qa + 8 * TC_PITCH + 16 * kk + 8);
                const uint32_t l0 = lds32(qb + 16 * kk), l1 = lds32(qb + 8 * TC_PITCH + 16 * kk), l2 = lds32(qb + 16 * kk + 8),
                               l3 = lds32(qb + 8 * TC_PITCH + 16 * kk + 8);
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    const __half* kr = ks + (32 * nh + 8 * nt + gq) * TC_PITCH + 16 * kk + 2 * t;
                    const uint32_t b0 = lds32(kr), b1 = lds32(kr + 8);
                    mma16816(s[nt], h0, h1, h2, h3, b0, b1);
                    mma16816(s[nt], l0, l1, l2, l3, b0, b1);
                }
            }
            // causal / range mask, then to shared memory
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int pair = 16 * mt + gq + 8 * (j >> 1), key = 32 * nh + 8 * nt + 2 * t + (j & 1);
                    const int row = pair / TC_GROUP;
                    const uint32_t kpos = p0 + key;
                    const bool ok = row < n_rows && kpos < n_pos && kpos <= start + (uint32_t)row;
                    sf[pair * TC_SP + key] = ok ? s[nt][j] : -INFINITY;
                }
        }
        __syncthreads();
        // ---- online softmax: warp w owns queries 8 w .. 8 w + 7 ----
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int pair = 8 * warp + i;
            const float s0 = sf[pair * TC_SP + lane], s1 = sf[pair * TC_SP + lane + 32];
            const float mc = warp_max(fmaxf(s0, s1));
            const float m_old = m_run[pair];
            const float m_new = fmaxf(m_old, mc);
            float e0 = 0.f, e1 = 0.f, a = 1.f;
            if (m_new > -INFINITY) {
                a = m_old > -INFINITY ? expf(m_old - m_new) : 0.f;
                e0 = s0 > -INFINITY ? expf(s0 - m_new) : 0.f;
                e1 = s1 > -INFINITY ? expf(s1 - m_new) : 0.f;
            }
            const float sum = warp_sum(e0 + e1);
            const __half h0 = __float2half_rn(e0), h1 = __float2half_rn(e1);
            p_hi[pair * TC_PP + lane] = h0;
            p_hi[pair * TC_PP + lane + 32] = h1;
            p_lo[pair * TC_PP + lane] = __float2half_rn(e0 - __half2float(h0));
            p_lo[pair * TC_PP + lane + 32] = __float2half_rn(e1 - __half2float(h1));
            if (lane == 0) {
                m_run[pair] = m_new;
                l_run[pair] = fmaf(l_run[pair], a, sum);
                alpha[pair] = a;
            }
        }
        __syncthreads();
        // ---- O = O * alpha + P V for queries 16 mt .. +15, head dims 64 nh .. +63 ----
        {
            const float a0 = alpha[16 * mt + gq], a1 = alpha[16 * mt + gq + 8];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) { o[nt][0] *= a0; o[nt][1] *= a0; o[nt][2] *= a1; o[nt][3] *= a1; }
            const __half* pa = p_hi + (16 * mt + gq) * TC_PP + 2 * t;
            const __half* pb = p_lo + (16 * mt + gq) * TC_PP + 2 * t;
#pragma unroll
            for (int kk = 0; kk < ATTN_CHUNK / 16; ++kk) {
                const uint32_t h0 = lds32(pa + 16 * kk), h1 = lds32(pa + 8 * TC_PP + 16 * kk), h2 = lds32(pa + 16 * kk + 8),
                               h3 = lds32(pa + 8 * TC_PP + 16 * kk + 8);
                const uint32_t l0 = lds32(pb + 16 * kk), l1 = lds32(pb + 8 * TC_PP + 16 * kk), l2 = lds32(pb + 16 * kk + 8),
                               l3 = lds32(pb + 8 * TC_PP + 16 * kk + 8);
#pragma unroll
                for (int np = 0; np < 4; ++np) {   // two 8-wide dim tiles per ldmatrix.x4
                    // lanes 0-15: keys 16 kk + lane of dims d0 .. d0 + 7; lanes 16-31: the same keys of dims d0 + 8 .. d0 + 15
                    const int d0 = 64 * nh + 16 * np;
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, vs + (16 * kk + (lane & 15)) * TC_PITCH + d0 + 8 * (lane >> 4));
                    mma16816(o[2 * np], h0, h1, h2, h3, b[0], b[1]);
                    mma16816(o[2 * np], l0, l1, l2, l3, b[0], b[1]);
                    mma16816(o[2 * np + 1], h0, h1, h2, h3, b[2], b[3]);
                    mma16816(o[2 * np + 1], l0, l1, l2, l3, b[2], b[3]);
                }
            }
        }
    }
    __syncthreads();
    // ---- one record per (span, kv head, query): [m, l, O[128]] ----
    float* rec0 = partials + ((uint64_t)span * g.n_kv + kvh) * TC_Q * (TC_HD + 2);
    if (threadIdx.x < TC_Q) {
        rec0[threadIdx.x * (TC_HD + 2)] = m_run[threadIdx.x];
        rec0[threadIdx.x * (TC_HD + 2) + 1] = l_run[threadIdx.x];
    }
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
        const int d = 64 * nh + 8 * nt + 2 * t;
        float* r0 = rec0 + (16 * mt + gq) * (TC_HD + 2) + 2 + d;
        float* r1 = rec0 + (16 * mt + gq + 8) * (TC_HD + 2) + 2 + d;
        r0[0] = o[nt][0]; r0[1] = o[nt][1];
        r1[0] = o[nt][2]; r1[1] = o[nt][3];
    }
}

bool attn_tc_supported(const AttnGeom& g, bool kv_f16) { return kv_f16 && g.hd == TC_HD && g.n_q / g.n_kv == TC_GROUP; }

// chunks per span from the session's KV capacity only (never from the call): enough spans to fill the GPU twice
int attn_tc_chunks_per_span(const AttnGeom& g, uint32_t kv_capacity) {
    const uint64_t cap_chunks = ((uint64_t)kv_capacity + ATTN_CHUNK - 1) / ATTN_CHUNK;
    uint64_t b = (cap_chunks * g.n_kv + 4 * 148 - 1) / (4 * 148);
    if (b < 1) b = 1;
    if (b > 64) b = 64;
    return (int)b;
}

dfl_status launch_attn_span_tc(cudaStream_t st, const AttnGeom& g, const float* q_rot, const void* k_cache, const void* v_cache,
                               uint32_t start, int n_rows, float* partials, int chunks_per_span) {
    static bool set = false;
    if (!set) {
        DFL_CUDA(cudaFuncSetAttribute(attn_span_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM));
        set = true;
    }
    const int n_chunks = (int)((start + (uint32_t)n_rows + ATTN_CHUNK - 1) / ATTN_CHUNK);
    const int n_spans = (n_chunks + chunks_per_span - 1) / chunks_per_span;
    launch_kf(4, attn_span_tc_kernel, dim3((unsigned)n_spans, (unsigned)g.n_kv), dim3(256), (size_t)TC_SMEM, st, g, q_rot,
              reinterpret_cast<const __half*>(k_cache), reinterpret_cast<const __half*>(v_cache), start, n_rows, partials, chunks_per_span);
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

}  // namespace dfl
