// Few-row (<= 16 activation rows) weight-streaming GEMM  y[r, o] = sum_i x[r, i] W[o, i]
// for quantised W, the B200 counterpart of the reference's
// kernel_mat_mat_*_fewrow_gen_* family (kernels/mat_mat_fewrow_gen.metal:374-474) and its
// routing (crates/qwen-llm/src/metal_forward/dispatch.rs:345-760).
//
// Design (HBM-bound: every weight byte is read exactly once):
//   * one CTA owns a 128-row tile and a contiguous range of 256-column blocks; a producer
//     warp streams the tile stages with 1-D bulk copies (TMA) into a multi-stage shared-memory
//     ring guarded by mbarriers, weights first (they do not depend on the previous kernel,
//     so under programmatic dependent launch they prefetch while it still runs), the packed
//     activations after griddepcontrol.wait;
//   * sixteen consumer warps: warp (ks, mh) owns columns [32 ks, 32 ks + 32) of the stage and
//     the four 16-row m-tiles 4 mh .. 4 mh + 3.  The *integer* quants go straight from shared
//     memory through a few logic ops into f16 MMA A-fragments (magic-number int->half
//     conversion, exact), the activations are the B operand as an exact hi+lo f16 pair, and
//     mma.sync m16n8k16 accumulates sum(x*q) in f32, two m-tiles interleaved so that four
//     independent accumulator chains are in flight.  Block scales (d*sc, dmin*m) are applied
//     in f32 per 16/32 columns, so no dequantised weight is ever rounded: a one-hot activation
//     row reproduces ggml's decoded weight bit for bit;
//   * per-warp partial tiles are summed in a fixed order through shared memory and the
//     split-K partial [16][n_out] is written coalesced.  No atomics: results are
//     deterministic and each activation row's result is independent of the other rows.
#include <vector>

#include "gemm_ts.cuh"

namespace dfl {

constexpr int K_SLICES = 8;                                         // warps along the 256 columns of a stage
constexpr int M_HALVES = 2;                                         // warps along the 128 rows
constexpr int CONSUMER_WARPS = K_SLICES * M_HALVES;                 // 16
constexpr int GEMM_THREADS = CONSUMER_WARPS * 32;                   // thread 0 also issues the bulk copies
constexpr int RED_LD = TILE_R + 4;                                  // padded row length of the reduce buffer
constexpr int WARP_SCRATCH = (TILE_R / M_HALVES) * 8;               // float2 per row of the warp's 64 rows

struct GemmParams {
    const uint8_t* w;
    const uint8_t* acts;
    float* out;
    const float* sumsq;
    int n_sumsq;
    float norm_k, eps, out_scale;
    int kblocks, splits;
    int row_tiles, ctas_per_split;
    uint32_t n_out;   // rows of this matrix
    uint32_t ld_out;  // row length of the partial buffer (>= n_out when several matrices share it)
    int* err;
};

__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_bf16(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t h2_sub(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("sub.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t h2_fma(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
constexpr uint32_t H2_1024 = 0x64006400u;   // half2(1024, 1024)
constexpr uint32_t H2_1056 = 0x64206420u;   // half2(1056, 1056)
constexpr uint32_t H2_1152 = 0x64806480u;   // half2(1152, 1152)
constexpr uint32_t H2_16TH = 0x2c002c00u;   // half2(1/16, 1/16)
constexpr uint32_t H2_M64 = 0xd400d400u;    // half2(-64, -64)
constexpr uint32_t H2_M96 = 0xd600d600u;    // half2(-96, -96)

// Activation fragments of one consumer warp for one stage (f16 hi/lo variant).
struct ActFrag16 {
    uint4 hi0, hi1, lo0, lo1;  // token g / g+8; .x,.y = step 0 (b0,b1); .z,.w = step 1
    __device__ __forceinline__ void load(const uint8_t* ast, int ks, int g, int t) {
        const int off = (32 * ks + 8 * t) * 2;
        hi0 = *reinterpret_cast<const uint4*>(ast + g * (ACT_ROW_HALFS * 2) + off);
        hi1 = *reinterpret_cast<const uint4*>(ast + (g + 8) * (ACT_ROW_HALFS * 2) + off);
        lo0 = *reinterpret_cast<const uint4*>(ast + ACT_PLANE + g * (ACT_ROW_HALFS * 2) + off);
        lo1 = *reinterpret_cast<const uint4*>(ast + ACT_PLANE + (g + 8) * (ACT_ROW_HALFS * 2) + off);
    }
};

// A[m][0..3] = step-0 fragment (a0,a1,a2,a3) of m-tile m, A[m][4..7] = step-1 fragment.
// Both steps into the same accumulators d[m][token half]: four independent chains of four MMAs.
__device__ __forceinline__ void mma_pair_same_scale(float (&d)[2][2][4], const uint32_t (&A)[2][8], const ActFrag16& f) {
#pragma unroll
    for (int m = 0; m < 2; ++m) {
        mma_f16(d[m][0], A[m][0], A[m][1], A[m][2], A[m][3], f.hi0.x, f.hi0.y);
        mma_f16(d[m][1], A[m][0], A[m][1], A[m][2], A[m][3], f.hi1.x, f.hi1.y);
    }
#pragma unroll
    for (int m = 0; m < 2; ++m) {
        mma_f16(d[m][0], A[m][4], A[m][5], A[m][6], A[m][7], f.hi0.z, f.hi0.w);
        mma_f16(d[m][1], A[m][4], A[m][5], A[m][6], A[m][7], f.hi1.z, f.hi1.w);
    }
#ifndef DFL_EXP_NOLO
#pragma unroll
    for (int m = 0; m < 2; ++m) {
        mma_f16(d[m][0], A[m][0], A[m][1], A[m][2], A[m][3], f.lo0.x, f.lo0.y);
        mma_f16(d[m][1], A[m][0], A[m][1], A[m][2], A[m][3], f.lo1.x, f.lo1.y);
    }
#pragma unroll
    for (int m = 0; m < 2; ++m) {
        mma_f16(d[m][0], A[m][4], A[m][5], A[m][6], A[m][7], f.lo0.z, f.lo0.w);
        mma_f16(d[m][1], A[m][4], A[m][5], A[m][6], A[m][7], f.lo1.z, f.lo1.w);
    }
#endif
}
// Separate accumulators per step (per-16-column scales): d[m][step][token half].
__device__ __forceinline__ void mma_pair_step_scale(float (&d)[2][2][2][4], const uint32_t (&A)[2][8], const ActFrag16& f) {
#pragma unroll
    for (int m = 0; m < 2; ++m) {
        mma_f16(d[m][0][0], A[m][0], A[m][1], A[m][2], A[m][3], f.hi0.x, f.hi0.y);
        mma_f16(d[m][0][1], A[m][0], A[m][1], A[m][2], A[m][3], f.hi1.x, f.hi1.y);
        mma_f16(d[m][1][0], A[m][4], A[m][5], A[m][6], A[m][7], f.hi0.z, f.hi0.w);
        mma_f16(d[m][1][1], A[m][4], A[m][5], A[m][6], A[m][7], f.hi1.z, f.hi1.w);
    }
#ifndef DFL_EXP_NOLO
#pragma unroll
    for (int m = 0; m < 2; ++m) {
        mma_f16(d[m][0][0], A[m][0], A[m][1], A[m][2], A[m][3], f.lo0.x, f.lo0.y);
        mma_f16(d[m][0][1], A[m][0], A[m][1], A[m][2], A[m][3], f.lo1.x, f.lo1.y);
        mma_f16(d[m][1][0], A[m][4], A[m][5], A[m][6], A[m][7], f.lo0.z, f.lo0.w);
        mma_f16(d[m][1][1], A[m][4], A[m][5], A[m][6], A[m][7], f.lo1.z, f.lo1.w);
    }
#endif
}

// acc[mt][c] (mt = 0..3 local m-tile of this warp): c0,c1 = (row 16mt+g, tokens 2t,2t+1),
// c2,c3 = (row 16mt+g+8, same tokens), c4..c7 the same for tokens 8+2t, 9+2t.
// sa / sb: (scale, min) of rows g / g+8;  s0..s3: activation sub-block sums of the lane's four tokens.
__device__ __forceinline__ void apply_scale_min(float (&acc)[8], const float (&d0)[4], const float (&d1)[4], float2 sa, float2 sb,
                                                float s0, float s1, float s2, float s3) {
    acc[0] = fmaf(-sa.y, s0, fmaf(sa.x, d0[0], acc[0]));
    acc[1] = fmaf(-sa.y, s1, fmaf(sa.x, d0[1], acc[1]));
    acc[2] = fmaf(-sb.y, s0, fmaf(sb.x, d0[2], acc[2]));
    acc[3] = fmaf(-sb.y, s1, fmaf(sb.x, d0[3], acc[3]));
    acc[4] = fmaf(-sa.y, s2, fmaf(sa.x, d1[0], acc[4]));
    acc[5] = fmaf(-sa.y, s3, fmaf(sa.x, d1[1], acc[5]));
    acc[6] = fmaf(-sb.y, s2, fmaf(sb.x, d1[2], acc[6]));
    acc[7] = fmaf(-sb.y, s3, fmaf(sb.x, d1[3], acc[7]));
}
// K-quant header {f16 d, f16 dmin, 12 B of 6-bit (scale, min)} -> (d*sc, dmin*m) of sub-block j.
__device__ __forceinline__ float2 k4_header_scale(const uint4 h, int j) {
    const float d = __half2float(__ushort_as_half((unsigned short)(h.x & 0xffffu)));
    const float dmin = __half2float(__ushort_as_half((unsigned short)(h.x >> 16)));
    uint32_t s, m;
    if (j < 4) {
        s = (h.y >> (8 * j)) & 63u;
        m = (h.z >> (8 * j)) & 63u;
    } else {
        const int jj = j - 4;
        s = ((h.w >> (8 * jj)) & 0xfu) | (((h.y >> (8 * jj + 6)) & 3u) << 4);
        m = ((h.w >> (8 * jj + 4)) & 0xfu) | (((h.z >> (8 * jj + 6)) & 3u) << 4);
    }
    return make_float2(d * (float)s, dmin * (float)m);
}

template <int DT>
struct Fmt;

template <>
struct Fmt<DFL_Q4_K> {
    static constexpr int STAGE = STAGE_Q4_K, ACT = ACT16_CHUNK, STAGES = 4, KC = 6;
    __device__ static __forceinline__ void unpack(uint32_t wq, uint32_t wq8, uint32_t (&A)[8]) {
        A[0] = h2_sub((wq & 0x000f000fu) | H2_1024, H2_1024);
        A[1] = h2_sub((wq8 & 0x000f000fu) | H2_1024, H2_1024);
        A[2] = h2_fma((wq & 0x00f000f0u) | H2_1024, H2_16TH, H2_M64);
        A[3] = h2_fma((wq8 & 0x00f000f0u) | H2_1024, H2_16TH, H2_M64);
        const uint32_t v = wq >> 8, v8 = wq8 >> 8;
        A[4] = h2_sub((v & 0x000f000fu) | H2_1024, H2_1024);
        A[5] = h2_sub((v8 & 0x000f000fu) | H2_1024, H2_1024);
        A[6] = h2_fma((v & 0x00f000f0u) | H2_1024, H2_16TH, H2_M64);
        A[7] = h2_fma((v8 & 0x00f000f0u) | H2_1024, H2_16TH, H2_M64);
    }
    __device__ static __forceinline__ void consume(const uint8_t* wst, const uint8_t* ast, float2* sc, float (&acc)[4][8], int ks,
                                                   int mh, int lane) {
        const int g = lane >> 2, t = lane & 3;
        // (d*sc, dmin*m) of this warp's 32-column sub-block for its 64 rows
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int r = lane + 32 * i;
            sc[r] = k4_header_scale(reinterpret_cast<const uint4*>(wst)[64 * mh + r], ks);
        }
        __syncwarp();
        ActFrag16 f;
        f.load(ast, ks, g, t);
        const float* S = reinterpret_cast<const float*>(ast + 2 * ACT_PLANE);
        const float s0 = S[(2 * t) * 8 + ks], s1 = S[(2 * t + 1) * 8 + ks], s2 = S[(2 * t + 8) * 8 + ks], s3 = S[(2 * t + 9) * 8 + ks];
        const uint4* q = reinterpret_cast<const uint4*>(wst + Q4K_OFF_QS) + (ks * 4 + 2 * mh) * 32 + lane;
#pragma unroll
        for (int p = 0; p < 2; ++p) {
            const uint4 qq = q[p * 32];  // x,y = m-tile 2p rows g,g+8;  z,w = m-tile 2p+1
            uint32_t A[2][8];
            unpack(qq.x, qq.y, A[0]);
            unpack(qq.z, qq.w, A[1]);
            float d[2][2][4] = {};
            mma_pair_same_scale(d, A, f);
#pragma unroll
            for (int m = 0; m < 2; ++m) {
                const int mt = 2 * p + m;
                apply_scale_min(acc[mt], d[m][0], d[m][1], sc[16 * mt + g], sc[16 * mt + g + 8], s0, s1, s2, s3);
            }
        }
        __syncwarp();
    }
};

template <>
struct Fmt<DFL_Q5_K> {
    static constexpr int STAGE = STAGE_Q5_K, ACT = ACT16_CHUNK, STAGES = 3, KC = 6;
    __device__ static __forceinline__ void unpack(uint32_t wq, uint32_t hb, uint32_t& a_l0, uint32_t& a_h0, uint32_t& a_l1, uint32_t& a_h1) {
        const uint32_t X = (hb & 0xfu) | ((hb & 0xf0u) << 12);
        const uint32_t v = wq >> 8;
        a_l0 = h2_sub((wq & 0x000f000fu) | ((X << 4) & 0x00100010u) | H2_1024, H2_1024);
        a_h0 = h2_fma((wq & 0x00f000f0u) | ((X << 7) & 0x01000100u) | H2_1024, H2_16TH, H2_M64);
        a_l1 = h2_sub((v & 0x000f000fu) | ((X << 2) & 0x00100010u) | H2_1024, H2_1024);
        a_h1 = h2_fma((v & 0x00f000f0u) | ((X << 5) & 0x01000100u) | H2_1024, H2_16TH, H2_M64);
    }
    __device__ static __forceinline__ void consume(const uint8_t* wst, const uint8_t* ast, float2* sc, float (&acc)[4][8], int ks,
                                                   int mh, int lane) {
        const int g = lane >> 2, t = lane & 3;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int r = lane + 32 * i;
            sc[r] = k4_header_scale(reinterpret_cast<const uint4*>(wst)[64 * mh + r], ks);
        }
        __syncwarp();
        ActFrag16 f;
        f.load(ast, ks, g, t);
        const float* S = reinterpret_cast<const float*>(ast + 2 * ACT_PLANE);
        const float s0 = S[(2 * t) * 8 + ks], s1 = S[(2 * t + 1) * 8 + ks], s2 = S[(2 * t + 8) * 8 + ks], s3 = S[(2 * t + 9) * 8 + ks];
        const uint4* q = reinterpret_cast<const uint4*>(wst + Q5K_OFF_QS) + (ks * 4 + 2 * mh) * 32 + lane;
        const uint32_t* qh = reinterpret_cast<const uint32_t*>(wst + Q5K_OFF_QH) + (ks * 4 + 2 * mh) * 32 + lane;
#pragma unroll
        for (int p = 0; p < 2; ++p) {
            const uint4 qq = q[p * 32];
            const uint32_t hb4 = qh[p * 32];  // bytes: (mt 2p, g), (mt 2p, g+8), (mt 2p+1, g), (mt 2p+1, g+8)
            uint32_t A[2][8];
            unpack(qq.x, hb4 & 0xffu, A[0][0], A[0][2], A[0][4], A[0][6]);
            unpack(qq.y, (hb4 >> 8) & 0xffu, A[0][1], A[0][3], A[0][5], A[0][7]);
            unpack(qq.z, (hb4 >> 16) & 0xffu, A[1][0], A[1][2], A[1][4], A[1][6]);
            unpack(qq.w, hb4 >> 24, A[1][1], A[1][3], A[1][5], A[1][7]);
            float d[2][2][4] = {};
            mma_pair_same_scale(d, A, f);
#pragma unroll
            for (int m = 0; m < 2; ++m) {
                const int mt = 2 * p + m;
                apply_scale_min(acc[mt], d[m][0], d[m][1], sc[16 * mt + g], sc[16 * mt + g + 8], s0, s1, s2, s3);
            }
        }
        __syncwarp();
    }
};

template <>
struct Fmt<DFL_Q6_K> {
    static constexpr int STAGE = STAGE_Q6_K, ACT = ACT16_CHUNK, STAGES = 3, KC = 6;
    // wq: low nibbles, X: the 2-bit high fields spread as byte0 -> bits 0-7, byte1 -> bits 16-23
    __device__ static __forceinline__ void unpack(uint32_t wq, uint32_t X, uint32_t& a_l0, uint32_t& a_h0, uint32_t& a_l1, uint32_t& a_h1) {
        const uint32_t v = wq >> 8;
        a_l0 = h2_sub((wq & 0x000f000fu) | ((X << 4) & 0x00300030u) | H2_1024, H2_1056);
        a_h0 = h2_fma((wq & 0x00f000f0u) | ((X << 6) & 0x03000300u) | H2_1024, H2_16TH, H2_M96);
        a_l1 = h2_sub((v & 0x000f000fu) | (X & 0x00300030u) | H2_1024, H2_1056);
        a_h1 = h2_fma((v & 0x00f000f0u) | ((X << 2) & 0x03000300u) | H2_1024, H2_16TH, H2_M96);
    }
    __device__ static __forceinline__ void consume(const uint8_t* wst, const uint8_t* ast, float2* sc, float (&acc)[4][8], int ks,
                                                   int mh, int lane) {
        const int g = lane >> 2, t = lane & 3;
        // d*sc of the two 16-column sub-blocks (2ks, 2ks+1) this warp owns, for its 64 rows
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int r = lane + 32 * i, row = 64 * mh + r;
            const uint16_t two = *reinterpret_cast<const uint16_t*>(wst + row * 16 + 2 * ks);
            const float d = __half2float(__ushort_as_half(reinterpret_cast<const uint16_t*>(wst + Q6K_OFF_D)[row]));
            sc[r] = make_float2(d * (float)(int8_t)(two & 0xff), d * (float)(int8_t)(two >> 8));
        }
        __syncwarp();
        ActFrag16 f;
        f.load(ast, ks, g, t);
        const uint4* ql = reinterpret_cast<const uint4*>(wst + Q6K_OFF_QL) + (ks * 4 + 2 * mh) * 32 + lane;
        const uint2* qh = reinterpret_cast<const uint2*>(wst + Q6K_OFF_QH) + (ks * 4 + 2 * mh) * 32 + lane;
#pragma unroll
        for (int p = 0; p < 2; ++p) {
            const uint4 qq = ql[p * 32];
            const uint2 hh = qh[p * 32];  // x: m-tile 2p (row g low 16 bits, row g+8 high 16 bits), y: m-tile 2p+1
            uint32_t A[2][8];
            unpack(qq.x, prmt(hh.x, 0u, 0x4140u), A[0][0], A[0][2], A[0][4], A[0][6]);
            unpack(qq.y, prmt(hh.x, 0u, 0x4342u), A[0][1], A[0][3], A[0][5], A[0][7]);
            unpack(qq.z, prmt(hh.y, 0u, 0x4140u), A[1][0], A[1][2], A[1][4], A[1][6]);
            unpack(qq.w, prmt(hh.y, 0u, 0x4342u), A[1][1], A[1][3], A[1][5], A[1][7]);
            float d[2][2][2][4] = {};
            mma_pair_step_scale(d, A, f);
#pragma unroll
            for (int m = 0; m < 2; ++m) {
                const int mt = 2 * p + m;
                const float2 sa = sc[16 * mt + g], sb = sc[16 * mt + g + 8];
                float(&a)[8] = acc[mt];
                a[0] = fmaf(sa.y, d[m][1][0][0], fmaf(sa.x, d[m][0][0][0], a[0]));
                a[1] = fmaf(sa.y, d[m][1][0][1], fmaf(sa.x, d[m][0][0][1], a[1]));
                a[2] = fmaf(sb.y, d[m][1][0][2], fmaf(sb.x, d[m][0][0][2], a[2]));
                a[3] = fmaf(sb.y, d[m][1][0][3], fmaf(sb.x, d[m][0][0][3], a[3]));
                a[4] = fmaf(sa.y, d[m][1][1][0], fmaf(sa.x, d[m][0][1][0], a[4]));
                a[5] = fmaf(sa.y, d[m][1][1][1], fmaf(sa.x, d[m][0][1][1], a[5]));
                a[6] = fmaf(sb.y, d[m][1][1][2], fmaf(sb.x, d[m][0][1][2], a[6]));
                a[7] = fmaf(sb.y, d[m][1][1][3], fmaf(sb.x, d[m][0][1][3], a[7]));
            }
        }
        __syncwarp();
    }
};

template <>
struct Fmt<DFL_Q8_0> {
    static constexpr int STAGE = STAGE_Q8_0, ACT = ACT16_CHUNK, STAGES = 3, KC = 4;
    __device__ static __forceinline__ void consume(const uint8_t* wst, const uint8_t* ast, float2* sc, float (&acc)[4][8], int ks,
                                                   int mh, int lane) {
        const int g = lane >> 2, t = lane & 3;
        float* scf = reinterpret_cast<float*>(sc);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int r = lane + 32 * i;
            scf[r] = __half2float(__ushort_as_half(reinterpret_cast<const uint16_t*>(wst)[(64 * mh + r) * 8 + ks]));
        }
        __syncwarp();
        ActFrag16 f;
        f.load(ast, ks, g, t);
        const uint4* q = reinterpret_cast<const uint4*>(wst + Q80_OFF_QS) + (ks * 8 + 4 * mh) * 32 + lane;
#pragma unroll
        for (int p = 0; p < 2; ++p) {
            uint32_t A[2][8];
#pragma unroll
            for (int m = 0; m < 2; ++m) {
                const uint4 qq = q[(2 * p + m) * 32];  // x: row g step0, y: row g step1, z: row g+8 step0, w: row g+8 step1
                A[m][0] = h2_sub(prmt(qq.x, H2_1024, 0x5150u), H2_1152);
                A[m][1] = h2_sub(prmt(qq.z, H2_1024, 0x5150u), H2_1152);
                A[m][2] = h2_sub(prmt(qq.x, H2_1024, 0x5352u), H2_1152);
                A[m][3] = h2_sub(prmt(qq.z, H2_1024, 0x5352u), H2_1152);
                A[m][4] = h2_sub(prmt(qq.y, H2_1024, 0x5150u), H2_1152);
                A[m][5] = h2_sub(prmt(qq.w, H2_1024, 0x5150u), H2_1152);
                A[m][6] = h2_sub(prmt(qq.y, H2_1024, 0x5352u), H2_1152);
                A[m][7] = h2_sub(prmt(qq.w, H2_1024, 0x5352u), H2_1152);
            }
            float d[2][2][4] = {};
            mma_pair_same_scale(d, A, f);
#pragma unroll
            for (int m = 0; m < 2; ++m) {
                const int mt = 2 * p + m;
                const float da = scf[16 * mt + g], db = scf[16 * mt + g + 8];
                float(&a)[8] = acc[mt];
                a[0] = fmaf(da, d[m][0][0], a[0]);
                a[1] = fmaf(da, d[m][0][1], a[1]);
                a[2] = fmaf(db, d[m][0][2], a[2]);
                a[3] = fmaf(db, d[m][0][3], a[3]);
                a[4] = fmaf(da, d[m][1][0], a[4]);
                a[5] = fmaf(da, d[m][1][1], a[5]);
                a[6] = fmaf(db, d[m][1][2], a[6]);
                a[7] = fmaf(db, d[m][1][3], a[7]);
            }
        }
        __syncwarp();
    }
};

template <>
struct Fmt<DFL_BF16> {
    static constexpr int STAGE = STAGE_B16, ACT = ACTB3_CHUNK, STAGES = 2, KC = 2;
    __device__ static __forceinline__ void consume(const uint8_t* wst, const uint8_t* ast, float2*, float (&acc)[4][8], int ks, int mh,
                                                   int lane) {
        const int g = lane >> 2, t = lane & 3;
        const int off = (32 * ks + 8 * t) * 2;
        uint4 b0[3], b1[3];
#pragma unroll
        for (int pl = 0; pl < 3; ++pl) {
            b0[pl] = *reinterpret_cast<const uint4*>(ast + pl * ACT_PLANE + g * (ACT_ROW_HALFS * 2) + off);
            b1[pl] = *reinterpret_cast<const uint4*>(ast + pl * ACT_PLANE + (g + 8) * (ACT_ROW_HALFS * 2) + off);
        }
        const uint4* q = reinterpret_cast<const uint4*>(wst) + (ks * 8 + 4 * mh) * 64 + lane;
#pragma unroll
        for (int p = 0; p < 2; ++p) {
            uint4 ra[2], rb[2];  // rows g, g+8: x,y = step0 (e01,e23), z,w = step1
#pragma unroll
            for (int m = 0; m < 2; ++m) {
                ra[m] = q[(2 * p + m) * 64];
                rb[m] = q[(2 * p + m) * 64 + 32];
            }
#pragma unroll
            for (int pl = 0; pl < 3; ++pl) {
#pragma unroll
                for (int m = 0; m < 2; ++m) {
                    mma_bf16(&acc[2 * p + m][0], ra[m].x, rb[m].x, ra[m].y, rb[m].y, b0[pl].x, b0[pl].y);
                    mma_bf16(&acc[2 * p + m][4], ra[m].x, rb[m].x, ra[m].y, rb[m].y, b1[pl].x, b1[pl].y);
                }
#pragma unroll
                for (int m = 0; m < 2; ++m) {
                    mma_bf16(&acc[2 * p + m][0], ra[m].z, rb[m].z, ra[m].w, rb[m].w, b0[pl].z, b0[pl].w);
                    mma_bf16(&acc[2 * p + m][4], ra[m].z, rb[m].z, ra[m].w, rb[m].w, b1[pl].z, b1[pl].w);
                }
            }
        }
    }
};

constexpr int RED_HALF_BYTES = K_SLICES * (MAX_ROWS / 2) * RED_LD * 4;   // eight slices x eight tokens x 132 floats = 33792

template <int DT>
constexpr int gemm_smem_bytes() {
    return Fmt<DT>::KC * Fmt<DT>::ACT + Fmt<DT>::STAGES * Fmt<DT>::STAGE + RED_HALF_BYTES + CONSUMER_WARPS * WARP_SCRATCH + 128;
}

// One CTA = one split (a range of at most KC column blocks, whose packed activations stay
// resident in shared memory) and every `ctas_per_split`-th row tile.  The weight stages of its
// tiles stream back to back through the ring, so the copy pipeline stays full across tile
// boundaries; after the last column block of a tile the eight column-slice partials are summed
// in a fixed order and the tile's [16][128] partial result is written.
template <int DT>
__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_fewrow_kernel(const GemmParams p) {
    using F = Fmt<DT>;
    constexpr int STAGES = F::STAGES;
    constexpr int OFF_RING = F::KC * F::ACT;
    constexpr int OFF_RED = OFF_RING + STAGES * F::STAGE;
    constexpr int OFF_SCR = OFF_RED + RED_HALF_BYTES;
    constexpr int OFF_BAR = OFF_SCR + CONSUMER_WARPS * WARP_SCRATCH;
    static_assert(OFF_BAR + 128 <= 227 * 1024, "shared memory budget");
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* acts_res = smem;
    uint8_t* ring = smem + OFF_RING;
    float* red = reinterpret_cast<float*>(smem + OFF_RED);
    float2* scratch = reinterpret_cast<float2*>(smem + OFF_SCR);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
    uint64_t* empty = full + STAGES;
    uint64_t* acts_bar = empty + STAGES;
    __shared__ float tok_scale[MAX_ROWS];
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sp = blockIdx.x % p.splits, c = blockIdx.x / p.splits;
    const int kb0 = (int)((long long)sp * p.kblocks / p.splits), kb1 = (int)((long long)(sp + 1) * p.kblocks / p.splits);
    const int n_kb = kb1 - kb0;
    const int n_my = (p.row_tiles - c + p.ctas_per_split - 1) / p.ctas_per_split;   // row tiles c, c + cps, ...
    const int n_it = n_my * n_kb;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], CONSUMER_WARPS);
        }
        mbar_init(acts_bar, 1);
        abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();
    // Let the next kernel in the stream start its own weight prefetch as early as possible.
    pdl_launch_dependents();

    float acc[4][8];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

    // Thread 0 doubles as the producer.  (pt, pk) = tile / column block of the next stage to issue.
    const bool producer = threadIdx.x == 0;
    const uint64_t tile_stride = (uint64_t)p.kblocks * F::STAGE;
    const uint8_t* wbase = p.w + (uint64_t)kb0 * F::STAGE;
    int pt = 0, pk = 0, issued = 0;
    auto issue = [&](int slot) {
        const uint8_t* src = wbase + (uint64_t)(c + pt * p.ctas_per_split) * tile_stride + (uint64_t)pk * F::STAGE;
        mbar_arrive_expect_tx(&full[slot], F::STAGE);
        bulk_g2s(ring + slot * F::STAGE, src, F::STAGE, &full[slot]);
        ++issued;
        if (++pk == n_kb) { pk = 0; ++pt; }
    };
    if (producer) {
        // weights do not depend on the previous kernel: the ring fills while that kernel still runs
        const int pre = n_it < STAGES ? n_it : STAGES;
        for (int i = 0; i < pre; ++i) issue(i);
        pdl_wait();
        mbar_arrive_expect_tx(acts_bar, (uint32_t)n_kb * F::ACT);
        for (int k = 0; k < n_kb; ++k)
            bulk_g2s(acts_res + k * F::ACT, p.acts + (uint64_t)(kb0 + k) * F::ACT, F::ACT, acts_bar);
    }

    const int ks = warp & (K_SLICES - 1), mh = warp >> 3;
    const int g = lane >> 2, t = lane & 3;
    float2* sc = scratch + warp * (TILE_R / M_HALVES);
    bool ok = n_it == 0 || mbar_wait_bounded(acts_bar, 0, p.err, DEV_ERR_WAIT_FULL);
    int kb = 0, tile = 0;
    for (int i = 0; i < n_it; ++i) {
        if (producer && ok && i >= 1 && issued < n_it) {
            const int j = i - 1, sj = j % STAGES;  // slot consumed in the previous iteration
            ok = mbar_wait_bounded(&empty[sj], (j / STAGES) & 1, p.err, DEV_ERR_WAIT_EMPTY);
            if (ok) issue(sj);
        }
        if (warp == 0) ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;  // the producer's outcome, warp-uniform
        const int s = i % STAGES;
        if (ok) ok = mbar_wait_bounded(&full[s], (i / STAGES) & 1, p.err, DEV_ERR_WAIT_FULL);
        if (ok) {
#ifndef DFL_EXP_NOCOMPUTE
            F::consume(ring + s * F::STAGE, acts_res + kb * F::ACT, sc, acc, ks, mh, lane);
#else
            acc[0][0] += reinterpret_cast<const float*>(ring + s * F::STAGE)[threadIdx.x];  // streaming-only experiment build
            __syncwarp();
#endif
            if (lane == 0) mbar_arrive(&empty[s]);
        } else {
            abort_flag = 1;  // keep walking the loop so that every warp meets the same barriers
        }
        if (++kb < n_kb) continue;
        kb = 0;

        // ---- tile finished: fixed-order sum over the eight column slices, tokens 0-7 then 8-15 ----
        if (tile == 0 && threadIdx.x < 256) {
            // per-token output scale; 16 threads per token add the sum-of-squares partials in a fixed tree
            const int tok = threadIdx.x >> 4, part = threadIdx.x & 15;
            float ss = 0.f;
            if (p.sumsq)
                for (int q = part; q < p.n_sumsq; q += 16) ss += p.sumsq[q * MAX_ROWS + tok];
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (part == 0) tok_scale[tok] = p.sumsq ? p.out_scale * (1.0f / sqrtf(ss / p.norm_k + p.eps)) : p.out_scale;
        }
        const uint32_t rt = (uint32_t)(c + tile * p.ctas_per_split);
        const int row = threadIdx.x & (TILE_R - 1), tq = threadIdx.x >> 7;
        const uint32_t orow = rt * TILE_R + row;
        float* dst = p.out + (uint64_t)sp * MAX_ROWS * p.ld_out + orow;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float* mine = red + ks * ((MAX_ROWS / 2) * RED_LD) + 64 * mh;
#pragma unroll
            for (int mt = 0; mt < 4; ++mt) {
                const int r0 = 16 * mt + g;
                mine[(2 * t) * RED_LD + r0] = acc[mt][4 * h + 0];
                mine[(2 * t + 1) * RED_LD + r0] = acc[mt][4 * h + 1];
                mine[(2 * t) * RED_LD + r0 + 8] = acc[mt][4 * h + 2];
                mine[(2 * t + 1) * RED_LD + r0 + 8] = acc[mt][4 * h + 3];
                acc[mt][4 * h + 0] = acc[mt][4 * h + 1] = acc[mt][4 * h + 2] = acc[mt][4 * h + 3] = 0.f;
            }
            __syncthreads();
            if (orow < p.n_out && !abort_flag) {
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int tl = 2 * tq + j, tok = 8 * h + tl;
                    float v = 0.f;
#pragma unroll
                    for (int wv = 0; wv < K_SLICES; ++wv) v += red[wv * ((MAX_ROWS / 2) * RED_LD) + tl * RED_LD + row];
                    dst[(uint64_t)tok * p.ld_out] = v * tok_scale[tok];
                }
            }
            __syncthreads();
        }
        ++tile;
    }
    __syncthreads();
    if (abort_flag && producer) {
        // Error word already set.  Give every copy this CTA armed a bounded chance to land before
        // the shared memory is released.
        for (int s = 0; s < STAGES; ++s) {
            uint32_t spins = 0;
            while (!mbar_try_wait(&full[s], 0) && !mbar_try_wait(&full[s], 1) && ++spins < (1u << 16)) __nanosleep(100);
        }
        uint32_t spins = 0;
        while (!mbar_try_wait(acts_bar, 0) && ++spins < (1u << 16)) __nanosleep(100);
    }
}

int gemm_max_kblocks_per_cta(int dtype) {
    switch (dtype) {
        case DFL_Q4_K: return Fmt<DFL_Q4_K>::KC;
        case DFL_Q5_K: return Fmt<DFL_Q5_K>::KC;
        case DFL_Q6_K: return Fmt<DFL_Q6_K>::KC;
        case DFL_Q8_0: return Fmt<DFL_Q8_0>::KC;
        case DFL_BF16: return Fmt<DFL_BF16>::KC;
        default: return 1;
    }
}

static int ctas_per_split(int row_tiles, int splits) {
    int cps = sm_count() / splits;
    if (cps < 1) cps = 1;
    return cps < row_tiles ? cps : row_tiles;
}

// Split count: every split must fit the resident activation window; beyond that, the count that
// minimises the longest CTA (rounds of row tiles x column blocks per split, plus a per-tile
// epilogue and a per-launch prologue measured in stage times).
int gemm_choose_splits(const QMatrix& m) {
    if (m.layout == LAYOUT_TS) {
        const int tiles = m.row_tiles;
        return m.dtype == DFL_BF16 ? gemm_tsb_choose_splits_multi(&tiles, 1, m.kblocks) : gemm_ts_choose_splits(m);
    }
    const int tiles = m.row_tiles > 0 ? m.row_tiles : 1;
    const int kc = gemm_max_kblocks_per_cta(m.dtype);
    const int s_min = (m.kblocks + kc - 1) / kc;
    int s_max = m.kblocks < 24 ? m.kblocks : 24;
    if (s_max < s_min) s_max = s_min;
    int best = s_min;
    double best_cost = 1e30;
    for (int s = s_min; s <= s_max; ++s) {
        const int cps = ctas_per_split(tiles, s);
        const int rounds = (tiles + cps - 1) / cps;
        const double unit = (double)((m.kblocks + s - 1) / s) + 1.0;
        const double cost = rounds * unit + 1.5 + 0.05 * s;
        if (cost < best_cost) { best_cost = cost; best = s; }
    }
    return best;
}

template <int DT>
static dfl_status launch_t(cudaStream_t st, const GemmParams& p, int grid, bool pdl) {
    static bool attr_set[16] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 16 && !attr_set[dev]) {
        DFL_CUDA(cudaFuncSetAttribute(gemm_fewrow_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, gemm_smem_bytes<DT>()));
        attr_set[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = gemm_smem_bytes<DT>();
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    DFL_CUDA(cudaLaunchKernelEx(&cfg, gemm_fewrow_kernel<DT>, p));
    count_launch();
    return DFL_OK;
}

// ---- optional per-launch timing ---------------------------------------------------------
struct TimedLaunch { cudaEvent_t e0, e1; uint64_t bytes; };
static bool g_timing = false;
static std::vector<TimedLaunch> g_timed;

static dfl_status launch_gemm_dispatch(cudaStream_t st, const QMatrix& m, const GemmParams& p, int grid, bool pdl) {
    switch (m.dtype) {
        case DFL_Q4_K: return launch_t<DFL_Q4_K>(st, p, grid, pdl);
        case DFL_Q5_K: return launch_t<DFL_Q5_K>(st, p, grid, pdl);
        case DFL_Q6_K: return launch_t<DFL_Q6_K>(st, p, grid, pdl);
        case DFL_Q8_0: return launch_t<DFL_Q8_0>(st, p, grid, pdl);
        case DFL_BF16: return launch_t<DFL_BF16>(st, p, grid, pdl);
        default: return fail(DFL_ERR_UNSUPPORTED, "gemm: weight dtype has no few-row kernel");
    }
}

dfl_status launch_gemm_fewrow(cudaStream_t st, const QMatrix& m, const uint8_t* acts, float* out, int splits,
                              const GemmEpilogue& ep, int* dev_err, bool pdl, uint32_t ld_out) {
    if (splits < 1 || splits > m.kblocks) return fail(DFL_ERR_BAD_ARG, "gemm: bad split count");
    if (m.layout == LAYOUT_TS) {
        auto* launch = m.dtype == DFL_BF16 ? launch_gemm_tsb : launch_gemm_ts;
        if (!g_timing) return launch(st, m, acts, out, splits, ep, dev_err, pdl, ld_out);
        TimedLaunch t{};
        t.bytes = m.ggml_bytes();
        DFL_CUDA(cudaEventCreate(&t.e0));
        DFL_CUDA(cudaEventCreate(&t.e1));
        DFL_CUDA(cudaEventRecord(t.e0, st));
        dfl_status rc = launch(st, m, acts, out, splits, ep, dev_err, pdl, ld_out);
        DFL_CUDA(cudaEventRecord(t.e1, st));
        g_timed.push_back(t);
        return rc;
    }
    GemmParams p;
    p.w = m.tiles;
    p.acts = acts;
    p.out = out;
    p.sumsq = ep.sumsq;
    p.n_sumsq = ep.n_sumsq;
    p.norm_k = ep.norm_k;
    p.eps = ep.eps;
    p.out_scale = ep.out_scale;
    p.kblocks = m.kblocks;
    p.splits = splits;
    p.n_out = (uint32_t)m.n_out;
    p.ld_out = ld_out ? ld_out : (uint32_t)m.n_out;
    p.err = dev_err;
    if ((m.kblocks + splits - 1) / splits > gemm_max_kblocks_per_cta(m.dtype))
        return fail(DFL_ERR_BAD_ARG, "gemm: too few splits for the resident activation window");
    p.row_tiles = m.row_tiles;
    p.ctas_per_split = ctas_per_split(m.row_tiles, splits);
    const int grid = p.ctas_per_split * splits;
    if (!g_timing) return launch_gemm_dispatch(st, m, p, grid, pdl);
    TimedLaunch t{};
    t.bytes = m.ggml_bytes();
    DFL_CUDA(cudaEventCreate(&t.e0));
    DFL_CUDA(cudaEventCreate(&t.e1));
    DFL_CUDA(cudaEventRecord(t.e0, st));
    dfl_status rc = launch_gemm_dispatch(st, m, p, grid, pdl);
    DFL_CUDA(cudaEventRecord(t.e1, st));
    g_timed.push_back(t);
    return rc;
}

// ---- activation packing (standalone; the model path packs inside its glue kernels) ------------
// One CTA per 256-column block; thread = (token = tid/16, 16 consecutive columns).
template <bool BF3>
__global__ void prep_acts_kernel(const float* __restrict__ x, int ld, int n_rows, float pre_scale, uint8_t* __restrict__ acts,
                                 int* err) {
    constexpr int CH = BF3 ? ACTB3_CHUNK : ACT16_CHUNK;
    const int kb = blockIdx.x, tok = threadIdx.x >> 4, seg = threadIdx.x & 15;
    uint8_t* chunk = acts + (uint64_t)kb * CH;
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
    float sum = 0.f;
    bool over = false;
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) {
        const int k = seg * 16 + 4 * q4;
        const int pos = act_pos(k);
        if (!BF3) {
            uint16_t hi[4], lo[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float f = v[4 * q4 + e];
                over |= (fabsf(f) >= 65504.f) && (fabsf(f) < INFINITY);
                const __half h = __float2half_rn(f);
                hi[e] = __half_as_ushort(h);
                lo[e] = __half_as_ushort(__float2half_rn(f - __half2float(h)));
                sum += f;
            }
            *reinterpret_cast<uint2*>(chunk + (tok * ACT_ROW_HALFS + pos) * 2) =
                make_uint2((uint32_t)hi[0] | ((uint32_t)hi[1] << 16), (uint32_t)hi[2] | ((uint32_t)hi[3] << 16));
            *reinterpret_cast<uint2*>(chunk + ACT_PLANE + (tok * ACT_ROW_HALFS + pos) * 2) =
                make_uint2((uint32_t)lo[0] | ((uint32_t)lo[1] << 16), (uint32_t)lo[2] | ((uint32_t)lo[3] << 16));
        } else {
            uint16_t b[3][4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float f = v[4 * q4 + e];
#pragma unroll
                for (int pl = 0; pl < 3; ++pl) {
                    const __nv_bfloat16 h = __float2bfloat16_rn(f);
                    b[pl][e] = __bfloat16_as_ushort(h);
                    f -= __bfloat162float(h);
                }
            }
#pragma unroll
            for (int pl = 0; pl < 3; ++pl)
                *reinterpret_cast<uint2*>(chunk + pl * ACT_PLANE + (tok * ACT_ROW_HALFS + pos) * 2) =
                    make_uint2((uint32_t)b[pl][0] | ((uint32_t)b[pl][1] << 16), (uint32_t)b[pl][2] | ((uint32_t)b[pl][3] << 16));
        }
    }
    if (!BF3) {
        // sum over the 32-column sub-block = this thread (16 columns) + its neighbour
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        if ((seg & 1) == 0) reinterpret_cast<float*>(chunk + 2 * ACT_PLANE)[tok * 8 + (seg >> 1)] = sum;
        if (over) atomicCAS(err, 0, DEV_ERR_OVERFLOW);
    }
}

dfl_status launch_prep_acts(cudaStream_t st, int weight_dtype, const float* x, int ld, int n_rows, uint64_t k, float pre_scale,
                            uint8_t* acts, int* dev_err) {
    if (k % TILE_K || n_rows < 0 || n_rows > MAX_ROWS) return fail(DFL_ERR_BAD_SHAPE, "prep_acts: shape");
    const unsigned grid = (unsigned)(k / TILE_K);
    if (dtype_uses_bf16_acts(weight_dtype)) prep_acts_kernel<true><<<grid, 256, 0, st>>>(x, ld, n_rows, pre_scale, acts, dev_err);
    else prep_acts_kernel<false><<<grid, 256, 0, st>>>(x, ld, n_rows, pre_scale, acts, dev_err);
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

dfl_status launch_prep_acts_for(cudaStream_t st, const QMatrix& m, const float* x, int ld, int n_rows, float pre_scale, uint8_t* acts,
                                int* dev_err) {
    if (m.layout == LAYOUT_TS && m.dtype == DFL_BF16) return launch_prep_acts_tsb(st, x, ld, n_rows, m.n_in, pre_scale, acts);
    if (m.layout == LAYOUT_TS) return launch_prep_acts_ts(st, x, ld, n_rows, m.n_in, pre_scale, acts, dev_err);
    return launch_prep_acts(st, m.dtype, x, ld, n_rows, m.n_in, pre_scale, acts, dev_err);
}

__global__ void reduce_partials_kernel(const float* part, int splits, int n_rows, uint64_t n_out, float* y,
                                       int ld_y, const int32_t* splits_dev) {
    pdl_prologue();
    if (splits_dev) splits += *splits_dev;
    const uint64_t o = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int r = blockIdx.y;
    if (o >= n_out || r >= n_rows) return;
    float v = 0.f;
    for (int s = 0; s < splits; ++s) v += part[((uint64_t)s * MAX_ROWS + r) * n_out + o];
    y[(uint64_t)r * ld_y + o] = v;
}

dfl_status launch_reduce_partials(cudaStream_t st, const float* part, int splits, int n_rows, uint64_t n_out, float* y, int ld_y,
                                  const int32_t* splits_dev) {
    dim3 grid((unsigned)((n_out + 255) / 256), (unsigned)n_rows);
    launch_k(reduce_partials_kernel, dim3(grid), dim3(256), 0, st, part, splits, n_rows, n_out, y, ld_y, splits_dev);
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

// ---- argmax + runner-up gap --------------------------------------------------
// Replaces kernel_argmax_top2_f32 (kernels/elementwise.metal:1231-1286) with the total-order,
// lowest-index tie rule of greedy_token (crates/qwen-llm/src/sampling.rs:1159-1181).
struct Top2 {
    int32_t k1, i1, k2, pad;  // total-order keys of best / runner-up, index of best
};
__device__ __forceinline__ void top2_push(Top2& a, int32_t key, int32_t idx) {
    if (key > a.k1 || (key == a.k1 && idx < a.i1)) { a.k2 = a.k1; a.k1 = key; a.i1 = idx; }
    else if (key > a.k2) a.k2 = key;
}
__device__ __forceinline__ void top2_merge(Top2& a, const Top2& b) {
    if (b.k1 > a.k1 || (b.k1 == a.k1 && b.i1 < a.i1)) {
        const int32_t second = a.k1 > b.k2 ? a.k1 : b.k2;
        a.k2 = second; a.k1 = b.k1; a.i1 = b.i1;
    } else {
        const int32_t second = b.k1 > a.k2 ? b.k1 : a.k2;
        a.k2 = second;
    }
}
__device__ __forceinline__ Top2 top2_warp_reduce(Top2 a) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Top2 b;
        b.k1 = __shfl_xor_sync(0xffffffffu, a.k1, o);
        b.i1 = __shfl_xor_sync(0xffffffffu, a.i1, o);
        b.k2 = __shfl_xor_sync(0xffffffffu, a.k2, o);
        top2_merge(a, b);
    }
    return a;
}
__device__ __forceinline__ Top2 top2_block_reduce(Top2 a) {
    __shared__ Top2 sh[32];
    a = top2_warp_reduce(a);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    if (lane == 0) sh[warp] = a;
    __syncthreads();
    if (warp == 0) {
        a = lane < nw ? sh[lane] : Top2{INT32_MIN, INT32_MAX, INT32_MIN, 0};
        a = top2_warp_reduce(a);
    }
    return a;
}
__device__ __forceinline__ float key_to_float(int32_t k) { return __int_as_float(k < 0 ? (k ^ 0x7fffffff) : k); }

__global__ void argmax_part_kernel(const float* logits, uint64_t vocab, uint64_t ld, Top2* parts) {
    pdl_prologue();
    const int row = blockIdx.y, part = blockIdx.x;
    const uint64_t per = (vocab + ARGMAX_PARTS - 1) / ARGMAX_PARTS;
    const uint64_t lo = part * per, hi = lo + per < vocab ? lo + per : vocab;
    Top2 a{INT32_MIN, INT32_MAX, INT32_MIN, 0};
    for (uint64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float v = logits[row * ld + i];
        // NaN sorts above everything so that it is reported (the host maps it to NanLogit)
        const int32_t key = (v != v) ? INT32_MAX : total_order_key(v);
        top2_push(a, key, (int32_t)i);
    }
    a = top2_block_reduce(a);
    if (threadIdx.x == 0) parts[row * ARGMAX_PARTS + part] = a;
}
// The same over split-K partial sums: each element is first reduced over the slices (slice order, as
// reduce_partials_kernel does) and written to `logits`, so the head's logits are produced and ranked in one pass.
__global__ void argmax_part_reduce_kernel(const float* part, int splits, uint64_t vocab, float* logits, uint64_t ld, Top2* parts) {
    pdl_prologue();
    const int row = blockIdx.y, pt = blockIdx.x;
    const uint64_t per = (vocab + ARGMAX_PARTS - 1) / ARGMAX_PARTS;
    const uint64_t lo = pt * per, hi = lo + per < vocab ? lo + per : vocab;
    Top2 a{INT32_MIN, INT32_MAX, INT32_MIN, 0};
    const uint64_t slice = (uint64_t)MAX_ROWS * vocab;
    for (uint64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float* src = part + (uint64_t)row * vocab + i;
        float v = 0.f;
        for (int s0 = 0; s0 < splits; s0 += 4) {   // four slices in flight per round trip, added in slice order
            float t[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) t[u] = __ldcg(src + (uint64_t)(s0 + u < splits ? s0 + u : splits - 1) * slice);
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (s0 + u < splits) v += t[u];
        }
        logits[row * ld + i] = v;
        const int32_t key = (v != v) ? INT32_MAX : total_order_key(v);
        top2_push(a, key, (int32_t)i);
    }
    a = top2_block_reduce(a);
    if (threadIdx.x == 0) parts[row * ARGMAX_PARTS + pt] = a;
}
__global__ void argmax_final_kernel(const Top2* parts, int32_t* argmax, float* gap) {
    pdl_prologue();
    const int row = blockIdx.x;
    Top2 a = threadIdx.x < ARGMAX_PARTS ? parts[row * ARGMAX_PARTS + threadIdx.x] : Top2{INT32_MIN, INT32_MAX, INT32_MIN, 0};
    a = top2_block_reduce(a);
    if (threadIdx.x == 0) {
        if (a.k1 == INT32_MAX) {  // NaN met: encode like GreedySelection::NanLogit (sampling.rs:283-293)
            argmax[row] = ~a.i1;
            gap[row] = 0.f;
        } else {
            argmax[row] = a.i1;
            gap[row] = a.k2 == INT32_MIN ? 0.f : key_to_float(a.k1) - key_to_float(a.k2);
        }
    }
}

dfl_status launch_argmax_top2(cudaStream_t st, const float* logits, int n_rows, uint64_t vocab, uint64_t ld, int32_t* argmax,
                              float* gap, void* scratch) {
    if (n_rows < 1 || vocab == 0) return fail(DFL_ERR_BAD_SHAPE, "argmax: shape");
    launch_k(argmax_part_kernel, dim3(dim3(ARGMAX_PARTS, n_rows)), dim3(256), 0, st, logits, vocab, ld, reinterpret_cast<Top2*>(scratch));
    launch_k(argmax_final_kernel, dim3(n_rows), dim3(64), 0, st, reinterpret_cast<const Top2*>(scratch), argmax, gap);
    count_launch(2);
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

dfl_status launch_reduce_argmax_top2(cudaStream_t st, const float* part, int splits, int n_rows, uint64_t vocab, float* logits, uint64_t ld,
                                     int32_t* argmax, float* gap, void* scratch) {
    if (n_rows < 1 || vocab == 0 || splits < 1) return fail(DFL_ERR_BAD_SHAPE, "argmax: shape");
    launch_k(argmax_part_reduce_kernel, dim3(dim3(ARGMAX_PARTS, n_rows)), dim3(256), 0, st, part, splits, vocab, logits, ld, reinterpret_cast<Top2*>(scratch));
    launch_k(argmax_final_kernel, dim3(n_rows), dim3(64), 0, st, reinterpret_cast<const Top2*>(scratch), argmax, gap);
    count_launch(2);
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

}  // namespace dfl

extern "C" {
void dfl_gemm_timing_begin(void) {
    for (auto& t : dfl::g_timed) { cudaEventDestroy(t.e0); cudaEventDestroy(t.e1); }
    dfl::g_timed.clear();
    dfl::g_timing = true;
}
dfl_status dfl_gemm_timing_end(double* ms_total, uint64_t* n_launches, uint64_t* weight_bytes) {
    dfl::g_timing = false;
    double ms = 0;
    uint64_t bytes = 0;
    for (auto& t : dfl::g_timed) {
        float one = 0;
        cudaEventSynchronize(t.e1);
        if (cudaEventElapsedTime(&one, t.e0, t.e1) == cudaSuccess) ms += one;
        bytes += t.bytes;
        cudaEventDestroy(t.e0);
        cudaEventDestroy(t.e1);
    }
    if (ms_total) *ms_total = ms;
    if (n_launches) *n_launches = dfl::g_timed.size();
    if (weight_bytes) *weight_bytes = bytes;
    dfl::g_timed.clear();
    return DFL_OK;
}
}
