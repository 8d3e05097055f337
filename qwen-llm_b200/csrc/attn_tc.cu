// Verify attention over an fp16 KV cache stored as position-major rows, on the tensor cores through mma.sync
// (reference: kernel_attn_decode_* / attn_v4, kernels/attn_v4.metal:65-265; CPU oracle forward.rs:896-921).  Sessions
// whose capacity reaches 16384 positions store the cache as tiles and use the tcgen05 kernel of attn_t5.cu instead;
// this kernel serves the shorter ones, where a CTA sees one or two chunks and launch latency is what counts.
//
// One CTA = one KV head x one span of `chunks_per_span` 64-position chunks; all 16 block rows x the 4 query
// heads of the GQA group (64 queries) share every K/V byte the CTA reads.  Four warps, warp w owns queries
// 16 w .. 16 w + 15 against all 64 keys of a chunk and all 128 head dims, so scores, probabilities and the
// running (max, sum, output) never leave registers:
//   S = Q K^T   mma.sync m16n8k16, Q (pre-scaled by 1/sqrt(hd)) as an exact f16 hi + lo pair, K straight from the cache
//   online softmax per query row: quad shuffles only
//   O = O * alpha + P V   the score fragments re-packed as the A operand (f16 hi + lo), V through ldmatrix.trans
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
constexpr int TC_STAGE = 2 * ATTN_CHUNK * TC_PITCH;   // halfs per K + V stage
constexpr int TC_SMEM = (2 * TC_Q * TC_PITCH + 2 * TC_STAGE) * 2;   // 104448: two CTAs per SM

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
// (a, b) -> f16x2 of the values and f16x2 of what the rounding left over
__device__ __forceinline__ void split_pair(float a, float b, uint32_t& hi, uint32_t& lo) {
    const __half2 h = __floats2half2_rn(a, b);
    const float2 back = __half22float2(h);
    const __half2 l = __floats2half2_rn(a - back.x, b - back.y);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = *reinterpret_cast<const uint32_t*>(&l);
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// 16-byte asynchronous copy global -> shared; copies nothing and writes zeros when !valid
__device__ __forceinline__ void cp_async16_zfill(void* smem, const void* gmem, bool valid) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem)), "l"(gmem), "r"(valid ? 16 : 0) : "memory");
}
}  // namespace

__global__ void __launch_bounds__(128) attn_span_tc_kernel(AttnGeom g, const float* q_rot, const __half* k_cache, const __half* v_cache,
                                                           uint32_t start, int n_rows, float* partials, int chunks_per_span) {
    pdl_prologue();
    extern __shared__ __align__(16) uint8_t sm_raw[];
    __half* q_hi = reinterpret_cast<__half*>(sm_raw);           // [64][136]
    __half* q_lo = q_hi + TC_Q * TC_PITCH;
    __half* kv = q_lo + TC_Q * TC_PITCH;                        // [2 stages][K | V][64][136]

    const int span = blockIdx.x, kvh = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, t = lane & 3;
    const uint32_t n_pos = start + (uint32_t)n_rows;
    const int c_begin = span * chunks_per_span;
    int c_end = (int)((n_pos + ATTN_CHUNK - 1) / ATTN_CHUNK);
    if (c_end > c_begin + chunks_per_span) c_end = c_begin + chunks_per_span;

    // K / V rows of one chunk and head into a stage: 64 x 256 B each, 16 B per copy, zero beyond the last position
    auto fetch = [&](int c) {
        __half* kst = kv + (c & 1) * TC_STAGE;
        const uint32_t p0 = (uint32_t)c * ATTN_CHUNK;
#pragma unroll
        for (int i = 0; i < ATTN_CHUNK * 16 / 128; ++i) {
            const int idx = threadIdx.x + 128 * i, kp = idx >> 4, v16 = idx & 15;
            const bool in = p0 + kp < n_pos;
            const uint64_t off = ((uint64_t)(in ? p0 + kp : p0) * g.n_kv + kvh) * TC_HD + v16 * 8;
            cp_async16_zfill(kst + kp * TC_PITCH + v16 * 8, k_cache + off, in);
            cp_async16_zfill(kst + ATTN_CHUNK * TC_PITCH + kp * TC_PITCH + v16 * 8, v_cache + off, in);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (c_begin < c_end) fetch(c_begin);

    // queries: pair = row * 4 + head-in-group, scaled by log2(e) / sqrt(hd) (scores live in the exp2 domain), split
    // into an exact f16 hi + lo pair
    const float scale = 1.4426950408889634f / sqrtf((float)TC_HD);
    for (int idx = threadIdx.x; idx < TC_Q * (TC_HD / 4); idx += 128) {
        const int pair = idx / (TC_HD / 4), d4 = (idx % (TC_HD / 4)) * 4;
        const int row = pair / TC_GROUP, qh = kvh * TC_GROUP + pair % TC_GROUP;
        float4 q = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row < n_rows) q = *reinterpret_cast<const float4*>(q_rot + ((uint64_t)row * g.n_q + qh) * TC_HD + d4);
        uint32_t h01, l01, h23, l23;
        split_pair(q.x * scale, q.y * scale, h01, l01);
        split_pair(q.z * scale, q.w * scale, h23, l23);
        *reinterpret_cast<uint2*>(q_hi + pair * TC_PITCH + d4) = make_uint2(h01, h23);
        *reinterpret_cast<uint2*>(q_lo + pair * TC_PITCH + d4) = make_uint2(l01, l23);
    }

    // this thread's two query rows (fragment rows gq and gq + 8 of the warp's m-tile)
    const int pair0 = 16 * warp + gq, pair1 = pair0 + 8;
    const int row0 = pair0 / TC_GROUP, row1 = pair1 / TC_GROUP;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float o[16][4];
#pragma unroll
    for (int i = 0; i < 16; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][j] = 0.f;

    for (int c = c_begin; c < c_end; ++c) {
        const uint32_t p0 = (uint32_t)c * ATTN_CHUNK;
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();   // chunk c landed for every thread; the other stage is fully consumed (and the query planes written)
        if (c + 1 < c_end) fetch(c + 1);
        const __half* ks = kv + (c & 1) * TC_STAGE;
        const __half* vs = ks + ATTN_CHUNK * TC_PITCH;
        // ---- S = Q K^T: 16 queries x 64 keys per warp ----
        float s[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
        {
            const __half* qa = q_hi + (16 * warp + gq) * TC_PITCH + 2 * t;
            const __half* qb = q_lo + (16 * warp + gq) * TC_PITCH + 2 * t;
#pragma unroll
            for (int kk = 0; kk < TC_HD / 16; ++kk) {
                const uint32_t h0 = lds32(qa + 16 * kk), h1 = lds32(qa + 8 * TC_PITCH + 16 * kk), h2 = lds32(qa + 16 * kk + 8),
                               h3 = lds32(qa + 8 * TC_PITCH + 16 * kk + 8);
                const uint32_t e0 = lds32(qb + 16 * kk), e1 = lds32(qb + 8 * TC_PITCH + 16 * kk), e2 = lds32(qb + 16 * kk + 8),
                               e3 = lds32(qb + 8 * TC_PITCH + 16 * kk + 8);
#pragma unroll
                uint32_t b0[8], b1[8];
#pragma unroll
                for (int nt = 0; nt < 8; ++nt) {
                    const __half* kr = ks + (8 * nt + gq) * TC_PITCH + 16 * kk + 2 * t;
                    b0[nt] = lds32(kr);
                    b1[nt] = lds32(kr + 8);
                    mma16816(s[nt], h0, h1, h2, h3, b0[nt], b1[nt]);
                }
#pragma unroll
                for (int nt = 0; nt < 8; ++nt) mma16816(s[nt], e0, e1, e2, e3, b0[nt], b1[nt]);
            }
        }
        // ---- causal / range mask (only the chunks that reach past the block's first position need it) ----
        if (p0 + ATTN_CHUNK > start + 1) {
            // keys of this chunk visible to the row: indices below lim (row r sees positions <= start + r; rows
            // beyond the call see nothing)
            const int lim0 = row0 < n_rows ? (int)(start + (uint32_t)row0 + 1 - p0) : 0;
            const int lim1 = row1 < n_rows ? (int)(start + (uint32_t)row1 + 1 - p0) : 0;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int key = 8 * nt + 2 * t + j;
                    if (key >= lim0) s[nt][j] = -INFINITY;
                    if (key >= lim1) s[nt][2 + j] = -INFINITY;
                }
        }
        // ---- online softmax per query row, in registers ----
        float mc0 = -INFINITY, mc1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            mc0 = fmaxf(mc0, fmaxf(s[nt][0], s[nt][1]));
            mc1 = fmaxf(mc1, fmaxf(s[nt][2], s[nt][3]));
        }
        mc0 = fmaxf(mc0, __shfl_xor_sync(0xffffffffu, mc0, 1));
        mc0 = fmaxf(mc0, __shfl_xor_sync(0xffffffffu, mc0, 2));
        mc1 = fmaxf(mc1, __shfl_xor_sync(0xffffffffu, mc1, 1));
        mc1 = fmaxf(mc1, __shfl_xor_sync(0xffffffffu, mc1, 2));
        const float mn0 = fmaxf(m0, mc0), mn1 = fmaxf(m1, mc1);
        const float ms0 = mn0 > -INFINITY ? mn0 : 0.f, ms1 = mn1 > -INFINITY ? mn1 : 0.f;   // exp2(-inf - ms) = 0, never NaN
        const float a0 = ex2(m0 - ms0), a1 = ex2(m1 - ms1);
        float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                s[nt][j] = ex2(s[nt][j] - ms0);
                s[nt][2 + j] = ex2(s[nt][2 + j] - ms1);
                sum0 += s[nt][j];
                sum1 += s[nt][2 + j];
            }
        sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
        sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
        sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
        sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
        m0 = mn0; m1 = mn1;
        l0 = fmaf(l0, a0, sum0);
        l1 = fmaf(l1, a1, sum1);
        // ---- O = O * alpha + P V ----
#pragma unroll
        for (int nt = 0; nt < 16; ++nt) { o[nt][0] *= a0; o[nt][1] *= a0; o[nt][2] *= a1; o[nt][3] *= a1; }
#pragma unroll
        for (int kk = 0; kk < ATTN_CHUNK / 16; ++kk) {
            // A fragment of keys 16 kk .. 16 kk + 15 = score tiles 2 kk (k 0-7) and 2 kk + 1 (k 8-15)
            const uint32_t h0 = pack_h2(s[2 * kk][0], s[2 * kk][1]), h1 = pack_h2(s[2 * kk][2], s[2 * kk][3]);
            const uint32_t h2 = pack_h2(s[2 * kk + 1][0], s[2 * kk + 1][1]), h3 = pack_h2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int np = 0; np < 8; ++np) {   // two 8-wide dim tiles per ldmatrix.x4
                // lanes 0-15: keys 16 kk + lane of dims 16 np .. + 7; lanes 16-31: the same keys of dims 16 np + 8 .. + 15
                uint32_t b[4];
                ldmatrix_x4_trans(b, vs + (16 * kk + (lane & 15)) * TC_PITCH + 16 * np + 8 * (lane >> 4));
                mma16816(o[2 * np], h0, h1, h2, h3, b[0], b[1]);
                mma16816(o[2 * np + 1], h0, h1, h2, h3, b[2], b[3]);
            }
        }
    }
    // ---- one record per (span, kv head, query): [m, l, O[128]], m back in the natural-log domain ----
    float* rec0 = partials + (((uint64_t)span * g.n_kv + kvh) * TC_Q + pair0) * (TC_HD + 2);
    float* rec1 = rec0 + 8 * (TC_HD + 2);
    if (t == 0) {
        rec0[0] = m0 * 0.6931471805599453f; rec0[1] = l0;
        rec1[0] = m1 * 0.6931471805599453f; rec1[1] = l1;
    }
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
        const int d = 8 * nt + 2 * t;
        *reinterpret_cast<float2*>(rec0 + 2 + d) = make_float2(o[nt][0], o[nt][1]);
        *reinterpret_cast<float2*>(rec1 + 2 + d) = make_float2(o[nt][2], o[nt][3]);
    }
}

// ---- the drafter's attention on the same scheme -----------------------------------------------------------------------
// Queries = the block's noise rows; keys = the context cache (f32, from column ctx_begin) followed by the noise rows'
// own K / V; allowed(q, k) = (!causal || k_pos <= q_pos) && (window == 0 || |q_pos - k_pos| < window)
// (kernels/dflash_attn.metal:99-103).  The f32 rows are split into exact f16 hi + lo pairs while they are copied into
// shared memory (through registers: 2 CTAs per SM overlap each other's loads), so
//   S = Qh Kh + Ql Kh + Qh Kl,   O += P Vh + P Vl   (P rounded to f16 as in the verify kernel)
// keeps f32-class accuracy against the f32 cache.  Same record format and span rule as attn_span_tc_kernel.
constexpr int DTC_SMEM = 6 * TC_Q * TC_PITCH * 2 + ATTN_CHUNK * 4;   // Q hi/lo, K hi/lo, V hi/lo, key positions: 104704

__global__ void __launch_bounds__(128) dattn_span_tc_kernel(AttnGeom g, const float* q_rot, const float* k_ctx, const float* v_ctx,
                                                            const uint32_t* pos_ctx, int ctx_begin, int n_ctx, const float* k_noise,
                                                            const float* v_noise, uint32_t noise_start, int n_rows, int causal,
                                                            uint32_t window, float* partials, int chunks_per_span) {
    pdl_prologue();
    extern __shared__ __align__(16) uint8_t sm_raw[];
    __half* q_hi = reinterpret_cast<__half*>(sm_raw);
    __half* q_lo = q_hi + TC_Q * TC_PITCH;
    __half* k_hi = q_lo + TC_Q * TC_PITCH;
    __half* k_lo = k_hi + ATTN_CHUNK * TC_PITCH;
    __half* v_hi = k_lo + ATTN_CHUNK * TC_PITCH;
    __half* v_lo = v_hi + ATTN_CHUNK * TC_PITCH;
    uint32_t* kpos = reinterpret_cast<uint32_t*>(v_lo + ATTN_CHUNK * TC_PITCH);

    const int span = blockIdx.x, kvh = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, t = lane & 3;
    const int n_keys = n_ctx + n_rows;
    const int c_begin = span * chunks_per_span;
    int c_end = (n_keys + ATTN_CHUNK - 1) / ATTN_CHUNK;
    if (c_end > c_begin + chunks_per_span) c_end = c_begin + chunks_per_span;

    const float scale = 1.4426950408889634f / sqrtf((float)TC_HD);
    for (int idx = threadIdx.x; idx < TC_Q * (TC_HD / 4); idx += 128) {
        const int pair = idx / (TC_HD / 4), d4 = (idx % (TC_HD / 4)) * 4;
        const int row = pair / TC_GROUP, qh = kvh * TC_GROUP + pair % TC_GROUP;
        float4 q = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row < n_rows) q = *reinterpret_cast<const float4*>(q_rot + ((uint64_t)row * g.n_q + qh) * TC_HD + d4);
        uint32_t h01, l01, h23, l23;
        split_pair(q.x * scale, q.y * scale, h01, l01);
        split_pair(q.z * scale, q.w * scale, h23, l23);
        *reinterpret_cast<uint2*>(q_hi + pair * TC_PITCH + d4) = make_uint2(h01, h23);
        *reinterpret_cast<uint2*>(q_lo + pair * TC_PITCH + d4) = make_uint2(l01, l23);
    }
    const int pair0 = 16 * warp + gq, pair1 = pair0 + 8;
    const int row0 = pair0 / TC_GROUP, row1 = pair1 / TC_GROUP;
    const uint32_t qpos0 = noise_start + (uint32_t)row0, qpos1 = noise_start + (uint32_t)row1;
    const bool live0 = row0 < n_rows, live1 = row1 < n_rows;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float o[16][4];
#pragma unroll
    for (int i = 0; i < 16; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][j] = 0.f;

    float4 kk[8], vv[8];
    bool have_half = false;
    const uint64_t row_stride = (uint64_t)g.n_kv * TC_HD;
    auto load_half = [&](int chunk, int half) {
        const uint64_t base = ((uint64_t)(ctx_begin + chunk * ATTN_CHUNK) * g.n_kv + kvh) * TC_HD;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int idx = threadIdx.x + 128 * (8 * half + i), kp = idx >> 5, d4 = (idx & 31) * 4;
            kk[i] = *reinterpret_cast<const float4*>(k_ctx + base + kp * row_stride + d4);
            vv[i] = *reinterpret_cast<const float4*>(v_ctx + base + kp * row_stride + d4);
        }
    };
    auto store_half = [&](int half) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int idx = threadIdx.x + 128 * (8 * half + i), kp = idx >> 5, d4 = (idx & 31) * 4;
            uint32_t h01, l01, h23, l23;
            split_pair(kk[i].x, kk[i].y, h01, l01);
            split_pair(kk[i].z, kk[i].w, h23, l23);
            *reinterpret_cast<uint2*>(k_hi + kp * TC_PITCH + d4) = make_uint2(h01, h23);
            *reinterpret_cast<uint2*>(k_lo + kp * TC_PITCH + d4) = make_uint2(l01, l23);
            split_pair(vv[i].x, vv[i].y, h01, l01);
            split_pair(vv[i].z, vv[i].w, h23, l23);
            *reinterpret_cast<uint2*>(v_hi + kp * TC_PITCH + d4) = make_uint2(h01, h23);
            *reinterpret_cast<uint2*>(v_lo + kp * TC_PITCH + d4) = make_uint2(l01, l23);
        }
    };
    for (int c = c_begin; c < c_end; ++c) {
        const int j0 = c * ATTN_CHUNK;
        const int n_here = min(ATTN_CHUNK, n_keys - j0);
        __syncthreads();   // previous chunk fully consumed (and the query planes written)
        // K / V rows of the chunk: 64 x 512 B each, one float4 of K and of V per thread and step, split on the way in
        if (j0 + ATTN_CHUNK <= n_ctx) {
            // whole chunk inside the context: eight K and eight V loads in flight per thread before any of them is
            // split; the first half was requested before the previous chunk's MMAs when that chunk took this path
            if (!have_half) load_half(c, 0);
            store_half(0);
            load_half(c, 1);
            store_half(1);
        } else
#pragma unroll 4
        for (int i = 0; i < ATTN_CHUNK * 32 / 128; ++i) {
            const int idx = threadIdx.x + 128 * i, kp = idx >> 5, d4 = (idx & 31) * 4;
            float4 kk = make_float4(0.f, 0.f, 0.f, 0.f), vv = kk;
            if (kp < n_here) {
                const int j = j0 + kp;
                if (j < n_ctx) {
                    const uint64_t off = ((uint64_t)(ctx_begin + j) * g.n_kv + kvh) * TC_HD + d4;
                    kk = *reinterpret_cast<const float4*>(k_ctx + off);
                    vv = *reinterpret_cast<const float4*>(v_ctx + off);
                } else {
                    const uint64_t off = ((uint64_t)(j - n_ctx) * g.n_kv + kvh) * TC_HD + d4;
                    kk = *reinterpret_cast<const float4*>(k_noise + off);
                    vv = *reinterpret_cast<const float4*>(v_noise + off);
                }
            }
            uint32_t h01, l01, h23, l23;
            split_pair(kk.x, kk.y, h01, l01);
            split_pair(kk.z, kk.w, h23, l23);
            *reinterpret_cast<uint2*>(k_hi + kp * TC_PITCH + d4) = make_uint2(h01, h23);
            *reinterpret_cast<uint2*>(k_lo + kp * TC_PITCH + d4) = make_uint2(l01, l23);
            split_pair(vv.x, vv.y, h01, l01);
            split_pair(vv.z, vv.w, h23, l23);
            *reinterpret_cast<uint2*>(v_hi + kp * TC_PITCH + d4) = make_uint2(h01, h23);
            *reinterpret_cast<uint2*>(v_lo + kp * TC_PITCH + d4) = make_uint2(l01, l23);
        }
        have_half = c + 1 < c_end && (c + 2) * ATTN_CHUNK <= n_ctx;
        if (have_half) load_half(c + 1, 0);   // lands while this chunk's MMAs run
        if (threadIdx.x < ATTN_CHUNK) {
            const int j = j0 + (int)threadIdx.x;
            kpos[threadIdx.x] = j < n_ctx ? pos_ctx[ctx_begin + j] : noise_start + (uint32_t)(j - n_ctx);
        }
        __syncthreads();
        // ---- S = Qh Kh + Ql Kh + Qh Kl ----
        float s[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
        {
            const __half* qa = q_hi + (16 * warp + gq) * TC_PITCH + 2 * t;
            const __half* qb = q_lo + (16 * warp + gq) * TC_PITCH + 2 * t;
#pragma unroll
            for (int kk = 0; kk < TC_HD / 16; ++kk) {
                const uint32_t h0 = lds32(qa + 16 * kk), h1 = lds32(qa + 8 * TC_PITCH + 16 * kk), h2 = lds32(qa + 16 * kk + 8),
                               h3 = lds32(qa + 8 * TC_PITCH + 16 * kk + 8);
                const uint32_t e0 = lds32(qb + 16 * kk), e1 = lds32(qb + 8 * TC_PITCH + 16 * kk), e2 = lds32(qb + 16 * kk + 8),
                               e3 = lds32(qb + 8 * TC_PITCH + 16 * kk + 8);
                uint32_t b0[8], b1[8];
#pragma unroll
                for (int nt = 0; nt < 8; ++nt) {
                    const __half* kr = k_hi + (8 * nt + gq) * TC_PITCH + 16 * kk + 2 * t;
                    b0[nt] = lds32(kr);
                    b1[nt] = lds32(kr + 8);
                    mma16816(s[nt], h0, h1, h2, h3, b0[nt], b1[nt]);
                }
#pragma unroll
                for (int nt = 0; nt < 8; ++nt) mma16816(s[nt], e0, e1, e2, e3, b0[nt], b1[nt]);
#pragma unroll
                for (int nt = 0; nt < 8; ++nt) {
                    const __half* kr = k_lo + (8 * nt + gq) * TC_PITCH + 16 * kk + 2 * t;
                    mma16816(s[nt], h0, h1, h2, h3, lds32(kr), lds32(kr + 8));
                }
            }
        }
        // ---- mask by positions ----
        const bool plain = !causal && window == 0 && n_here == ATTN_CHUNK && live0 && live1;
        if (!plain) {
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int key = 8 * nt + 2 * t + j;
                    const uint32_t kp = kpos[key];
                    const bool in = key < n_here;
                    const uint32_t d0 = qpos0 > kp ? qpos0 - kp : kp - qpos0, d1 = qpos1 > kp ? qpos1 - kp : kp - qpos1;
                    const bool ok0 = live0 && in && (!causal || kp <= qpos0) && (window == 0 || d0 < window);
                    const bool ok1 = live1 && in && (!causal || kp <= qpos1) && (window == 0 || d1 < window);
                    if (!ok0) s[nt][j] = -INFINITY;
                    if (!ok1) s[nt][2 + j] = -INFINITY;
                }
        }
        // ---- online softmax per query row, in registers ----
        float mc0 = -INFINITY, mc1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            mc0 = fmaxf(mc0, fmaxf(s[nt][0], s[nt][1]));
            mc1 = fmaxf(mc1, fmaxf(s[nt][2], s[nt][3]));
        }
        mc0 = fmaxf(mc0, __shfl_xor_sync(0xffffffffu, mc0, 1));
        mc0 = fmaxf(mc0, __shfl_xor_sync(0xffffffffu, mc0, 2));
        mc1 = fmaxf(mc1, __shfl_xor_sync(0xffffffffu, mc1, 1));
        mc1 = fmaxf(mc1, __shfl_xor_sync(0xffffffffu, mc1, 2));
        const float mn0 = fmaxf(m0, mc0), mn1 = fmaxf(m1, mc1);
        const float ms0 = mn0 > -INFINITY ? mn0 : 0.f, ms1 = mn1 > -INFINITY ? mn1 : 0.f;
        const float a0 = ex2(m0 - ms0), a1 = ex2(m1 - ms1);
        float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                s[nt][j] = ex2(s[nt][j] - ms0);
                s[nt][2 + j] = ex2(s[nt][2 + j] - ms1);
                sum0 += s[nt][j];
                sum1 += s[nt][2 + j];
            }
        sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
        sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
        sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
        sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
        m0 = mn0; m1 = mn1;
        l0 = fmaf(l0, a0, sum0);
        l1 = fmaf(l1, a1, sum1);
        // ---- O = O * alpha + P Vh + P Vl ----
#pragma unroll
        for (int nt = 0; nt < 16; ++nt) { o[nt][0] *= a0; o[nt][1] *= a0; o[nt][2] *= a1; o[nt][3] *= a1; }
#pragma unroll
        for (int kk = 0; kk < ATTN_CHUNK / 16; ++kk) {
            const uint32_t h0 = pack_h2(s[2 * kk][0], s[2 * kk][1]), h1 = pack_h2(s[2 * kk][2], s[2 * kk][3]);
            const uint32_t h2 = pack_h2(s[2 * kk + 1][0], s[2 * kk + 1][1]), h3 = pack_h2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int np = 0; np < 8; ++np) {
                uint32_t b[4], e[4];
                const int voff = (16 * kk + (lane & 15)) * TC_PITCH + 16 * np + 8 * (lane >> 4);
                ldmatrix_x4_trans(b, v_hi + voff);
                ldmatrix_x4_trans(e, v_lo + voff);
                mma16816(o[2 * np], h0, h1, h2, h3, b[0], b[1]);
                mma16816(o[2 * np + 1], h0, h1, h2, h3, b[2], b[3]);
                mma16816(o[2 * np], h0, h1, h2, h3, e[0], e[1]);
                mma16816(o[2 * np + 1], h0, h1, h2, h3, e[2], e[3]);
            }
        }
    }
    float* rec0 = partials + (((uint64_t)span * g.n_kv + kvh) * TC_Q + pair0) * (TC_HD + 2);
    float* rec1 = rec0 + 8 * (TC_HD + 2);
    if (t == 0) {
        rec0[0] = m0 * 0.6931471805599453f; rec0[1] = l0;
        rec1[0] = m1 * 0.6931471805599453f; rec1[1] = l1;
    }
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
        const int d = 8 * nt + 2 * t;
        *reinterpret_cast<float2*>(rec0 + 2 + d) = make_float2(o[nt][0], o[nt][1]);
        *reinterpret_cast<float2*>(rec1 + 2 + d) = make_float2(o[nt][2], o[nt][3]);
    }
}

bool dattn_tc_supported(const AttnGeom& g) { return g.hd == TC_HD && g.n_kv > 0 && g.n_q / g.n_kv == TC_GROUP; }

// launches the span kernel and returns the number of records per (kv head, query) the combine pass has to merge
dfl_status launch_dattn_span_tc(cudaStream_t st, const AttnGeom& g, const float* q_rot, const float* k_ctx, const float* v_ctx,
                                const uint32_t* pos_ctx, int ctx_begin, int n_ctx, const float* k_noise, const float* v_noise,
                                uint32_t noise_start, int n_rows, bool causal, uint32_t window, float* partials, uint32_t ctx_capacity,
                                int* n_spans_out) {
    static bool set = false;
    if (!set) {
        DFL_CUDA(cudaFuncSetAttribute(dattn_span_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DTC_SMEM));
        set = true;
    }
    const int cps = attn_tc_chunks_per_span(g, ctx_capacity + MAX_ROWS);
    const int n_chunks = (n_ctx + n_rows + ATTN_CHUNK - 1) / ATTN_CHUNK;
    const int n_spans = (n_chunks + cps - 1) / cps;
    launch_k(dattn_span_tc_kernel, dim3((unsigned)n_spans, (unsigned)g.n_kv), dim3(128), (size_t)DTC_SMEM, st, g, q_rot, k_ctx, v_ctx, pos_ctx,
              ctx_begin, n_ctx, k_noise, v_noise, noise_start, n_rows, causal ? 1 : 0, window, partials, cps);
    count_launch();
    DFL_CUDA(cudaGetLastError());
    *n_spans_out = n_spans;
    return DFL_OK;
}

bool attn_tc_supported(const AttnGeom& g, bool kv_f16) { return kv_f16 && g.hd == TC_HD && g.n_q / g.n_kv == TC_GROUP; }

// chunks per span from the session's KV capacity only (never from the call): two CTAs per SM, two waves
int attn_tc_chunks_per_span(const AttnGeom& g, uint32_t kv_capacity) {
    const uint64_t cap_chunks = ((uint64_t)kv_capacity + ATTN_CHUNK - 1) / ATTN_CHUNK;
    const uint64_t slots = 4ull * (uint64_t)sm_count();
    uint64_t b = (cap_chunks * g.n_kv + slots - 1) / slots;
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
    launch_k(attn_span_tc_kernel, dim3((unsigned)n_spans, (unsigned)g.n_kv), dim3(128), (size_t)TC_SMEM, st, g, q_rot,
              reinterpret_cast<const __half*>(k_cache), reinterpret_cast<const __half*>(v_cache), start, n_rows, partials, chunks_per_span);
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

}  // namespace dfl
