// Few-row (<= 16 activation rows) weight-streaming GEMM  y[r, o] = sum_i x[r, i] W[o, i]
// for quantised W, the B200 counterpart of the reference's
// kernel_mat_mat_*_fewrow_gen_* family (kernels/mat_mat_fewrow_gen.metal:374-474) and its
// routing (crates/qwen-llm/src/metal_forward/dispatch.rs:345-760).
//
// Design (HBM-bound: every weight byte is read exactly once):
//   * one CTA owns a 128-row tile and a contiguous range of 256-column blocks; a producer
//     warp streams the tile stages with 1-D bulk copies (TMA) into a 2-3 deep shared-memory
//     ring guarded by mbarriers, weights first (they do not depend on the previous kernel,
//     so under programmatic dependent launch they prefetch while it still runs), the packed
//     activations after griddepcontrol.wait;
//   * eight consumer warps split the 256 columns (32 each).  The *integer* quants go
//     straight from shared memory through a few logic ops into f16 MMA A-fragments
//     (magic-number int->half conversion, exact), the activations are the B operand as an
//     exact hi+lo f16 pair, and mma.sync m16n8k16 accumulates sum(x*q) in f32.  Block scales
//     (d*sc, dmin*m) are applied in f32 per 16/32 columns, so no dequantised weight is ever
//     rounded: a one-hot activation row reproduces ggml's decoded weight bit for bit;
//   * per-warp partial tiles are summed in a fixed order through shared memory and the
//     split-K partial [16][n_out] is written coalesced.  No atomics: results are
//     deterministic and each activation row's result is independent of the other rows.
#include <vector>

#include "tiles.cuh"

namespace dfl {

constexpr int CONSUMER_WARPS = 8;
constexpr int GEMM_THREADS = (CONSUMER_WARPS + 1) * 32;
constexpr int RED_LD = TILE_R + 4;                                  // padded row length of the reduce buffer
constexpr int RED_BYTES = CONSUMER_WARPS * MAX_ROWS * RED_LD * 4;   // 67584
constexpr int WARP_SCRATCH = TILE_R * 8;                            // float2 per row, per warp

struct GemmParams {
    const uint8_t* w;
    const uint8_t* acts;
    float* out;
    const float* sumsq;
    int n_sumsq;
    float norm_k, eps, out_scale;
    int kblocks, splits;
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
    __device__ __forceinline__ void load(const uint8_t* ast, int w, int g, int t) {
        const int off = (32 * w + 8 * t) * 2;
        hi0 = *reinterpret_cast<const uint4*>(ast + g * (ACT_ROW_HALFS * 2) + off);
        hi1 = *reinterpret_cast<const uint4*>(ast + (g + 8) * (ACT_ROW_HALFS * 2) + off);
        lo0 = *reinterpret_cast<const uint4*>(ast + ACT_PLANE + g * (ACT_ROW_HALFS * 2) + off);
        lo1 = *reinterpret_cast<const uint4*>(ast + ACT_PLANE + (g + 8) * (ACT_ROW_HALFS * 2) + off);
    }
};
// d0 += A(step) x tokens 0-7, d1 += A(step) x tokens 8-15, hi and lo parts.
__device__ __forceinline__ void mma_step0(float (&d0)[4], float (&d1)[4], const ActFrag16& f, uint32_t a0, uint32_t a1,
                                          uint32_t a2, uint32_t a3) {
    mma_f16(d0, a0, a1, a2, a3, f.hi0.x, f.hi0.y);
    mma_f16(d1, a0, a1, a2, a3, f.hi1.x, f.hi1.y);
    mma_f16(d0, a0, a1, a2, a3, f.lo0.x, f.lo0.y);
    mma_f16(d1, a0, a1, a2, a3, f.lo1.x, f.lo1.y);
}
__device__ __forceinline__ void mma_step1(float (&d0)[4], float (&d1)[4], const ActFrag16& f, uint32_t a0, uint32_t a1,
                                          uint32_t a2, uint32_t a3) {
    mma_f16(d0, a0, a1, a2, a3, f.hi0.z, f.hi0.w);
    mma_f16(d1, a0, a1, a2, a3, f.hi1.z, f.hi1.w);
    mma_f16(d0, a0, a1, a2, a3, f.lo0.z, f.lo0.w);
    mma_f16(d1, a0, a1, a2, a3, f.lo1.z, f.lo1.w);
}

// ---- per-format stage consumers ----------------------------------------------
// acc[mt][c]: c0,c1 = (row 16mt+g, tokens 2t,2t+1), c2,c3 = (row 16mt+g+8, same tokens),
//             c4..c7 the same for tokens 8+2t, 9+2t.
template <int DT>
struct Fmt;

template <>
struct Fmt<DFL_Q4_K> {
    static constexpr int STAGE = STAGE_Q4_K, ACT = ACT16_CHUNK, STAGES = 3;
    static constexpr bool HAS_HI = false;
    __device__ static __forceinline__ void consume(const uint8_t* wst, const uint8_t* ast, float2* sc, float (&acc)[8][8],
                                                   int w, int lane) {
        const int g = lane >> 2, t = lane & 3;
        // (d*sc_w, dmin*m_w) of this warp's 32-column sub-block for all 128 rows
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = lane + 32 * i;
            const uint4 h = reinterpret_cast<const uint4*>(wst)[r];
            const float d = __half2float(__ushort_as_half((unsigned short)(h.x & 0xffffu)));
            const float dmin = __half2float(__ushort_as_half((unsigned short)(h.x >> 16)));
            uint32_t s, m;
            if (w < 4) {
                s = (h.y >> (8 * w)) & 63u;
                m = (h.z >> (8 * w)) & 63u;
            } else {
                const int jj = w - 4;
                s = ((h.w >> (8 * jj)) & 0xfu) | (((h.y >> (8 * jj + 6)) & 3u) << 4);
                m = ((h.w >> (8 * jj + 4)) & 0xfu) | (((h.z >> (8 * jj + 6)) & 3u) << 4);
            }
            sc[r] = make_float2(d * (float)s, dmin * (float)m);
        }
        __syncwarp();
        ActFrag16 f;
        f.load(ast, w, g, t);
        const float* S = reinterpret_cast<const float*>(ast + 2 * ACT_PLANE);
        const float s0 = S[(2 * t) * 8 + w], s1 = S[(2 * t + 1) * 8 + w], s2 = S[(2 * t + 8) * 8 + w], s3 = S[(2 * t + 9) * 8 + w];
        const uint4* q = reinterpret_cast<const uint4*>(wst + Q4K_OFF_QS) + (w * 4) * 32 + lane;
#pragma unroll
        for (int mtp = 0; mtp < 4; ++mtp) {
            const uint4 qq = q[mtp * 32];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int mt = 2 * mtp + h;
                const uint32_t wg = h ? qq.z : qq.x, wg8 = h ? qq.w : qq.y;
                const uint32_t l0 = h2_sub((wg & 0x000f000fu) | H2_1024, H2_1024), l1 = h2_sub((wg8 & 0x000f000fu) | H2_1024, H2_1024);
                const uint32_t h0 = h2_fma((wg & 0x00f000f0u) | H2_1024, H2_16TH, H2_M64), h1 = h2_fma((wg8 & 0x00f000f0u) | H2_1024, H2_16TH, H2_M64);
                const uint32_t vg = wg >> 8, vg8 = wg8 >> 8;
                const uint32_t l2 = h2_sub((vg & 0x000f000fu) | H2_1024, H2_1024), l3 = h2_sub((vg8 & 0x000f000fu) | H2_1024, H2_1024);
                const uint32_t h2 = h2_fma((vg & 0x00f000f0u) | H2_1024, H2_16TH, H2_M64), h3 = h2_fma((vg8 & 0x00f000f0u) | H2_1024, H2_16TH, H2_M64);
                float d0[4] = {0.f, 0.f, 0.f, 0.f}, d1[4] = {0.f, 0.f, 0.f, 0.f};
                mma_step0(d0, d1, f, l0, l1, h0, h1);
                mma_step1(d0, d1, f, l2, l3, h2, h3);
                const float2 a = sc[16 * mt + g], b = sc[16 * mt + g + 8];
                acc[mt][0] = fmaf(-a.y, s0, fmaf(a.x, d0[0], acc[mt][0]));
                acc[mt][1] = fmaf(-a.y, s1, fmaf(a.x, d0[1], acc[mt][1]));
                acc[mt][2] = fmaf(-b.y, s0, fmaf(b.x, d0[2], acc[mt][2]));
                acc[mt][3] = fmaf(-b.y, s1, fmaf(b.x, d0[3], acc[mt][3]));
                acc[mt][4] = fmaf(-a.y, s2, fmaf(a.x, d1[0], acc[mt][4]));
                acc[mt][5] = fmaf(-a.y, s3, fmaf(a.x, d1[1], acc[mt][5]));
                acc[mt][6] = fmaf(-b.y, s2, fmaf(b.x, d1[2], acc[mt][6]));
                acc[mt][7] = fmaf(-b.y, s3, fmaf(b.x, d1[3], acc[mt][7]));
            }
        }
        __syncwarp();
    }
};

template <>
struct Fmt<DFL_Q5_K> {
    static constexpr int STAGE = STAGE_Q5_K, ACT = ACT16_CHUNK, STAGES = 2;
    __device__ static __forceinline__ void consume(const uint8_t* wst, const uint8_t* ast, float2* sc, float (&acc)[8][8],
                                                   int w, int lane) {
        const int g = lane >> 2, t = lane & 3;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = lane + 32 * i;
            const uint4 h = reinterpret_cast<const uint4*>(wst)[r];
            const float d = __half2float(__ushort_as_half((unsigned short)(h.x & 0xffffu)));
            const float dmin = __half2float(__ushort_as_half((unsigned short)(h.x >> 16)));
            uint32_t s, m;
            if (w < 4) {
                s = (h.y >> (8 * w)) & 63u;
                m = (h.z >> (8 * w)) & 63u;
            } else {
                const int jj = w - 4;
                s = ((h.w >> (8 * jj)) & 0xfu) | (((h.y >> (8 * jj + 6)) & 3u) << 4);
                m = ((h.w >> (8 * jj + 4)) & 0xfu) | (((h.z >> (8 * jj + 6)) & 3u) << 4);
            }
            sc[r] = make_float2(d * (float)s, dmin * (float)m);
        }
        __syncwarp();
        ActFrag16 f;
        f.load(ast, w, g, t);
        const float* S = reinterpret_cast<const float*>(ast + 2 * ACT_PLANE);
        const float s0 = S[(2 * t) * 8 + w], s1 = S[(2 * t + 1) * 8 + w], s2 = S[(2 * t + 8) * 8 + w], s3 = S[(2 * t + 9) * 8 + w];
        const uint4* q = reinterpret_cast<const uint4*>(wst + Q5K_OFF_QS) + (w * 4) * 32 + lane;
        const uint32_t* qh = reinterpret_cast<const uint32_t*>(wst + Q5K_OFF_QH) + (w * 4) * 32 + lane;
#pragma unroll
        for (int mtp = 0; mtp < 4; ++mtp) {
            const uint4 qq = q[mtp * 32];
            const uint32_t hb4 = qh[mtp * 32];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int mt = 2 * mtp + h;
                uint32_t a[2][4];  // [row half][l(step0), h(step0), l(step1), h(step1)]
#pragma unroll
                for (int rh = 0; rh < 2; ++rh) {
                    const uint32_t wq = h ? (rh ? qq.w : qq.z) : (rh ? qq.y : qq.x);
                    const uint32_t hb = (hb4 >> (8 * (2 * h + rh))) & 0xffu;
                    const uint32_t X = (hb & 0xfu) | ((hb & 0xf0u) << 12);
                    const uint32_t v = wq >> 8;
                    a[rh][0] = h2_sub((wq & 0x000f000fu) | ((X << 4) & 0x00100010u) | H2_1024, H2_1024);
                    a[rh][1] = h2_fma((wq & 0x00f000f0u) | ((X << 7) & 0x01000100u) | H2_1024, H2_16TH, H2_M64);
                    a[rh][2] = h2_sub((v & 0x000f000fu) | ((X << 2) & 0x00100010u) | H2_1024, H2_1024);
                    a[rh][3] = h2_fma((v & 0x00f000f0u) | ((X << 5) & 0x01000100u) | H2_1024, H2_16TH, H2_M64);
                }
                float d0[4] = {0.f, 0.f, 0.f, 0.f}, d1[4] = {0.f, 0.f, 0.f, 0.f};
                mma_step0(d0, d1, f, a[0][0], a[1][0], a[0][1], a[1][1]);
                mma_step1(d0, d1, f, a[0][2], a[1][2], a[0][3], a[1][3]);
                const float2 sa = sc[16 * mt + g], sb = sc[16 * mt + g + 8];
                acc[mt][0] = fmaf(-sa.y, s0, fmaf(sa.x, d0[0], acc[mt][0]));
                acc[mt][1] = fmaf(-sa.y, s1, fmaf(sa.x, d0[1], acc[mt][1]));
                acc[mt][2] = fmaf(-sb.y, s0, fmaf(sb.x, d0[2], acc[mt][2]));
                acc[mt][3] = fmaf(-sb.y, s1, fmaf(sb.x, d0[3], acc[mt][3]));
                acc[mt][4] = fmaf(-sa.y, s2, fmaf(sa.x, d1[0], acc[mt][4]));
                acc[mt][5] = fmaf(-sa.y, s3, fmaf(sa.x, d1[1], acc[mt][5]));
                acc[mt][6] = fmaf(-sb.y, s2, fmaf(sb.x, d1[2], acc[mt][6]));
                acc[mt][7] = fmaf(-sb.y, s3, fmaf(sb.x, d1[3], acc[mt][7]));
            }
        }
        __syncwarp();
    }
};

template <>
struct Fmt<DFL_Q6_K> {
    static constexpr int STAGE = STAGE_Q6_K, ACT = ACT16_CHUNK, STAGES = 2;
    __device__ static __forceinline__ void consume(const uint8_t* wst, const uint8_t* ast, float2* sc, float (&acc)[8][8],
                                                   int w, int lane) {
        const int g = lane >> 2, t = lane & 3;
        // d*sc of the two 16-column sub-blocks (2w, 2w+1) this warp owns
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = lane + 32 * i;
            const uint16_t two = *reinterpret_cast<const uint16_t*>(wst + r * 16 + 2 * w);
            const float d = __half2float(__ushort_as_half(reinterpret_cast<const uint16_t*>(wst + Q6K_OFF_D)[r]));
            sc[r] = make_float2(d * (float)(int8_t)(two & 0xff), d * (float)(int8_t)(two >> 8));
        }
        __syncwarp();
        ActFrag16 f;
        f.load(ast, w, g, t);
        const uint4* ql = reinterpret_cast<const uint4*>(wst + Q6K_OFF_QL) + (w * 4) * 32 + lane;
        const uint2* qh = reinterpret_cast<const uint2*>(wst + Q6K_OFF_QH) + (w * 4) * 32 + lane;
#pragma unroll
        for (int mtp = 0; mtp < 4; ++mtp) {
            const uint4 qq = ql[mtp * 32];
            const uint2 hh2 = qh[mtp * 32];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int mt = 2 * mtp + h;
                const uint32_t hh = h ? hh2.y : hh2.x;
                uint32_t a[2][4];
#pragma unroll
                for (int rh = 0; rh < 2; ++rh) {
                    const uint32_t wq = h ? (rh ? qq.w : qq.z) : (rh ? qq.y : qq.x);
                    const uint32_t X = prmt(hh, 0u, rh ? 0x4342u : 0x4140u);  // byte0 -> bits 0-7, byte1 -> bits 16-23
                    const uint32_t v = wq >> 8;
                    a[rh][0] = h2_sub((wq & 0x000f000fu) | ((X << 4) & 0x00300030u) | H2_1024, H2_1056);
                    a[rh][1] = h2_fma((wq & 0x00f000f0u) | ((X << 6) & 0x03000300u) | H2_1024, H2_16TH, H2_M96);
                    a[rh][2] = h2_sub((v & 0x000f000fu) | (X & 0x00300030u) | H2_1024, H2_1056);
                    a[rh][3] = h2_fma((v & 0x00f000f0u) | ((X << 2) & 0x03000300u) | H2_1024, H2_16TH, H2_M96);
                }
                float d00[4] = {0.f, 0.f, 0.f, 0.f}, d01[4] = {0.f, 0.f, 0.f, 0.f};
                float d10[4] = {0.f, 0.f, 0.f, 0.f}, d11[4] = {0.f, 0.f, 0.f, 0.f};
                mma_step0(d00, d01, f, a[0][0], a[1][0], a[0][1], a[1][1]);
                mma_step1(d10, d11, f, a[0][2], a[1][2], a[0][3], a[1][3]);
                const float2 sa = sc[16 * mt + g], sb = sc[16 * mt + g + 8];
                acc[mt][0] = fmaf(sa.y, d10[0], fmaf(sa.x, d00[0], acc[mt][0]));
                acc[mt][1] = fmaf(sa.y, d10[1], fmaf(sa.x, d00[1], acc[mt][1]));
                acc[mt][2] = fmaf(sb.y, d10[2], fmaf(sb.x, d00[2], acc[mt][2]));
                acc[mt][3] = fmaf(sb.y, d10[3], fmaf(sb.x, d00[3], acc[mt][3]));
                acc[mt][4] = fmaf(sa.y, d11[0], fmaf(sa.x, d01[0], acc[mt][4]));
                acc[mt][5] = fmaf(sa.y, d11[1], fmaf(sa.x, d01[1], acc[mt][5]));
                acc[mt][6] = fmaf(sb.y, d11[2], fmaf(sb.x, d01[2], acc[mt][6]));
                acc[mt][7] = fmaf(sb.y, d11[3], fmaf(sb.x, d01[3], acc[mt][7]));
            }
        }
        __syncwarp();
    }
};

template <>
struct Fmt<DFL_Q8_0> {
    static constexpr int STAGE = STAGE_Q8_0, ACT = ACT16_CHUNK, STAGES = 2;
    __device__ static __forceinline__ void consume(const uint8_t* wst, const uint8_t* ast, float2* sc, float (&acc)[8][8],
                                                   int w, int lane) {
        const int g = lane >> 2, t = lane & 3;
        float* scf = reinterpret_cast<float*>(sc);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = lane + 32 * i;
            scf[r] = __half2float(__ushort_as_half(reinterpret_cast<const uint16_t*>(wst)[r * 8 + w]));
        }
        __syncwarp();
        ActFrag16 f;
        f.load(ast, w, g, t);
        const uint4* q = reinterpret_cast<const uint4*>(wst + Q80_OFF_QS) + (w * 8) * 32 + lane;
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) {
            const uint4 qq = q[mt * 32];  // x: row g step0, y: row g step1, z: row g+8 step0, w: row g+8 step1
            const uint32_t a00 = h2_sub(prmt(qq.x, H2_1024, 0x5150u), H2_1152), a02 = h2_sub(prmt(qq.x, H2_1024, 0x5352u), H2_1152);
            const uint32_t a01 = h2_sub(prmt(qq.z, H2_1024, 0x5150u), H2_1152), a03 = h2_sub(prmt(qq.z, H2_1024, 0x5352u), H2_1152);
            const uint32_t a10 = h2_sub(prmt(qq.y, H2_1024, 0x5150u), H2_1152), a12 = h2_sub(prmt(qq.y, H2_1024, 0x5352u), H2_1152);
            const uint32_t a11 = h2_sub(prmt(qq.w, H2_1024, 0x5150u), H2_1152), a13 = h2_sub(prmt(qq.w, H2_1024, 0x5352u), H2_1152);
            float d0[4] = {0.f, 0.f, 0.f, 0.f}, d1[4] = {0.f, 0.f, 0.f, 0.f};
            mma_step0(d0, d1, f, a00, a01, a02, a03);
            mma_step1(d0, d1, f, a10, a11, a12, a13);
            const float da = scf[16 * mt + g], db = scf[16 * mt + g + 8];
            acc[mt][0] = fmaf(da, d0[0], acc[mt][0]);
            acc[mt][1] = fmaf(da, d0[1], acc[mt][1]);
            acc[mt][2] = fmaf(db, d0[2], acc[mt][2]);
            acc[mt][3] = fmaf(db, d0[3], acc[mt][3]);
            acc[mt][4] = fmaf(da, d1[0], acc[mt][4]);
            acc[mt][5] = fmaf(da, d1[1], acc[mt][5]);
            acc[mt][6] = fmaf(db, d1[2], acc[mt][6]);
            acc[mt][7] = fmaf(db, d1[3], acc[mt][7]);
        }
        __syncwarp();
    }
};

template <>
struct Fmt<DFL_BF16> {
    static constexpr int STAGE = STAGE_B16, ACT = ACTB3_CHUNK, STAGES = 2;
    __device__ static __forceinline__ void consume(const uint8_t* wst, const uint8_t* ast, float2*, float (&acc)[8][8], int w,
                                                   int lane) {
        const int g = lane >> 2, t = lane & 3;
        const int off = (32 * w + 8 * t) * 2;
        uint4 b0[3], b1[3];
#pragma unroll
        for (int p = 0; p < 3; ++p) {
            b0[p] = *reinterpret_cast<const uint4*>(ast + p * ACT_PLANE + g * (ACT_ROW_HALFS * 2) + off);
            b1[p] = *reinterpret_cast<const uint4*>(ast + p * ACT_PLANE + (g + 8) * (ACT_ROW_HALFS * 2) + off);
        }
        const uint4* q = reinterpret_cast<const uint4*>(wst) + (w * 8) * 64 + lane;
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) {
            const uint4 ra = q[mt * 64], rb = q[mt * 64 + 32];  // rows g, g+8: x,y = step0 (e01,e23), z,w = step1
#pragma unroll
            for (int p = 0; p < 3; ++p) {
                mma_bf16(&acc[mt][0], ra.x, rb.x, ra.y, rb.y, b0[p].x, b0[p].y);
                mma_bf16(&acc[mt][4], ra.x, rb.x, ra.y, rb.y, b1[p].x, b1[p].y);
                mma_bf16(&acc[mt][0], ra.z, rb.z, ra.w, rb.w, b0[p].z, b0[p].w);
                mma_bf16(&acc[mt][4], ra.z, rb.z, ra.w, rb.w, b1[p].z, b1[p].w);
            }
        }
    }
};

template <int DT>
constexpr int gemm_smem_bytes() {
    return Fmt<DT>::STAGES * (Fmt<DT>::STAGE + Fmt<DT>::ACT) + CONSUMER_WARPS * WARP_SCRATCH + 128;
}

template <int DT>
__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_fewrow_kernel(const GemmParams p) {
    using F = Fmt<DT>;
    constexpr int STAGES = F::STAGES;
    constexpr int SLOT = F::STAGE + F::ACT;
    static_assert(STAGES * SLOT >= RED_BYTES, "stage ring must be able to hold the reduce buffer");
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ring = smem;
    float2* scratch = reinterpret_cast<float2*>(smem + STAGES * SLOT);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * SLOT + CONSUMER_WARPS * WARP_SCRATCH);
    uint64_t* empty = full + STAGES;
    __shared__ float tok_scale[MAX_ROWS];
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rt = blockIdx.x / p.splits, sp = blockIdx.x % p.splits;
    const int kb0 = (int)((long long)sp * p.kblocks / p.splits), kb1 = (int)((long long)(sp + 1) * p.kblocks / p.splits);
    const int n_it = kb1 - kb0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], CONSUMER_WARPS);
        }
        abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();
    // Let the next kernel in the stream start its own weight prefetch as early as possible.
    pdl_launch_dependents();

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

    if (warp == CONSUMER_WARPS) {
        // ---------------- producer ----------------
        if (lane == 0) {
            const uint8_t* wsrc = p.w + ((uint64_t)rt * p.kblocks + kb0) * F::STAGE;
            const uint8_t* asrc = p.acts + (uint64_t)kb0 * F::ACT;
            const int pre = n_it < STAGES ? n_it : STAGES;
            // weights of the first stages do not depend on the previous kernel
            for (int i = 0; i < pre; ++i) {
                mbar_arrive_expect_tx(&full[i], F::STAGE + F::ACT);
                bulk_g2s(ring + i * SLOT, wsrc + (uint64_t)i * F::STAGE, F::STAGE, &full[i]);
            }
            pdl_wait();
            for (int i = 0; i < pre; ++i) bulk_g2s(ring + i * SLOT + F::STAGE, asrc + (uint64_t)i * F::ACT, F::ACT, &full[i]);
            bool ok = true;
            int issued = pre;
            for (int i = STAGES; i < n_it && ok; ++i) {
                const int s = i % STAGES;
                ok = mbar_wait_bounded(&empty[s], ((i / STAGES) - 1) & 1, p.err, DEV_ERR_WAIT_EMPTY);
                if (!ok) break;
                mbar_arrive_expect_tx(&full[s], F::STAGE + F::ACT);
                bulk_g2s(ring + s * SLOT, wsrc + (uint64_t)i * F::STAGE, F::STAGE, &full[s]);
                bulk_g2s(ring + s * SLOT + F::STAGE, asrc + (uint64_t)i * F::ACT, F::ACT, &full[s]);
                issued = i + 1;
            }
            if (!ok) {
                // Give the copies still in flight a bounded chance to land before the CTA exits.
                atomicExch(&abort_flag, 1);
                for (int i = issued > STAGES ? issued - STAGES : 0; i < issued; ++i)
                    mbar_wait_bounded(&full[i % STAGES], (i / STAGES) & 1, p.err, DEV_ERR_WAIT_DRAIN);
            }
        }
    } else {
        // ---------------- consumers ----------------
        float2* sc = scratch + warp * TILE_R;
        bool ok = true;
        for (int i = 0; i < n_it; ++i) {
            const int s = i % STAGES;
            ok = mbar_wait_bounded(&full[s], (i / STAGES) & 1, p.err, DEV_ERR_WAIT_FULL);
            if (!ok) break;
            F::consume(ring + s * SLOT, ring + s * SLOT + F::STAGE, sc, acc, warp, lane);
            if (lane == 0) mbar_arrive(&empty[s]);
        }
        if (!ok) atomicExch(&abort_flag, 1);
    }
    if (warp == CONSUMER_WARPS) pdl_wait();  // lanes 1..31 (and lane 0 again): harmless, keeps the wait on every path
    __syncthreads();
    if (abort_flag) return;  // error word already set; outputs are left untouched

    // ---------------- epilogue: fixed-order cross-warp sum ----------------
    float* red = reinterpret_cast<float*>(ring);
    if (warp < CONSUMER_WARPS) {
        const int g = lane >> 2, t = lane & 3;
        float* mine = red + warp * (MAX_ROWS * RED_LD);
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) {
            const int r0 = 16 * mt + g;
            mine[(2 * t) * RED_LD + r0] = acc[mt][0];
            mine[(2 * t + 1) * RED_LD + r0] = acc[mt][1];
            mine[(2 * t) * RED_LD + r0 + 8] = acc[mt][2];
            mine[(2 * t + 1) * RED_LD + r0 + 8] = acc[mt][3];
            mine[(2 * t + 8) * RED_LD + r0] = acc[mt][4];
            mine[(2 * t + 9) * RED_LD + r0] = acc[mt][5];
            mine[(2 * t + 8) * RED_LD + r0 + 8] = acc[mt][6];
            mine[(2 * t + 9) * RED_LD + r0 + 8] = acc[mt][7];
        }
    }
    if (threadIdx.x < MAX_ROWS) {
        float sc = p.out_scale;
        if (p.sumsq) {
            float ss = 0.f;
            for (int i = 0; i < p.n_sumsq; ++i) ss += p.sumsq[i * MAX_ROWS + threadIdx.x];
            sc *= 1.0f / sqrtf(ss / p.norm_k + p.eps);
        }
        tok_scale[threadIdx.x] = sc;
    }
    __syncthreads();
    if (threadIdx.x < 256) {
        const int row = threadIdx.x & (TILE_R - 1), th = threadIdx.x >> 7;
        const uint32_t orow = (uint32_t)rt * TILE_R + row;
        if (orow < p.n_out) {
            float* dst = p.out + (uint64_t)sp * MAX_ROWS * p.ld_out + orow;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int tok = th * 8 + j;
                float v = 0.f;
#pragma unroll
                for (int wv = 0; wv < CONSUMER_WARPS; ++wv) v += red[wv * (MAX_ROWS * RED_LD) + tok * RED_LD + row];
                dst[(uint64_t)tok * p.ld_out] = v * tok_scale[tok];
            }
        }
    }
}

int gemm_choose_splits(const QMatrix& m) {
    // Aim at roughly two co-resident CTAs per SM; never split finer than one block per CTA.
    constexpr int kTargetCtas = 2 * 148;
    int s = kTargetCtas / (m.row_tiles > 0 ? m.row_tiles : 1);
    if (s < 1) s = 1;
    if (s > m.kblocks) s = m.kblocks;
    if (s > 16) s = 16;
    return s;
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

static dfl_status launch_gemm_dispatch(cudaStream_t st, const QMatrix& m, const GemmParams& p, int grid, bool pdl);

dfl_status launch_gemm_fewrow(cudaStream_t st, const QMatrix& m, const uint8_t* acts, float* out, int splits,
                              const GemmEpilogue& ep, int* dev_err, bool pdl, uint32_t ld_out) {
    if (splits < 1 || splits > m.kblocks) return fail(DFL_ERR_BAD_ARG, "gemm: bad split count");
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
    const int grid = m.row_tiles * splits;
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

// ---- activation packing ------------------------------------------------------
// One CTA per 256-column block; thread = (token = tid/16, 16 consecutive columns).
template <bool BF3>
__global__ void prep_acts_kernel(const float* __restrict__ x, int ld, int n_rows, float pre_scale, uint8_t* __restrict__ acts,
                                 int* err) {
    constexpr int CH = BF3 ? ACTB3_CHUNK : ACT16_CHUNK;
    const int kb = blockIdx.x, tok = threadIdx.x >> 4, seg = threadIdx.x & 15;
    const int w = seg >> 1, s = seg & 1;
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
    if (!BF3) {
        float sum = 0.f;
        bool over = false;
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            __half hi[4], lo[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float f = v[4 * t + e];
                over |= (fabsf(f) >= 65504.f) && (fabsf(f) < INFINITY);
                hi[e] = __float2half_rn(f);
                lo[e] = __float2half_rn(f - __half2float(hi[e]));
                sum += f;
            }
            const int pos = 32 * w + 8 * t + 4 * s;
            uint2 ph, pl;
            ph.x = (uint32_t)__half_as_ushort(hi[0]) | ((uint32_t)__half_as_ushort(hi[1]) << 16);
            ph.y = (uint32_t)__half_as_ushort(hi[2]) | ((uint32_t)__half_as_ushort(hi[3]) << 16);
            pl.x = (uint32_t)__half_as_ushort(lo[0]) | ((uint32_t)__half_as_ushort(lo[1]) << 16);
            pl.y = (uint32_t)__half_as_ushort(lo[2]) | ((uint32_t)__half_as_ushort(lo[3]) << 16);
            *reinterpret_cast<uint2*>(chunk + (tok * ACT_ROW_HALFS + pos) * 2) = ph;
            *reinterpret_cast<uint2*>(chunk + ACT_PLANE + (tok * ACT_ROW_HALFS + pos) * 2) = pl;
        }
        // sum over the 32-column sub-block = this thread (16 columns) + its neighbour
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        if (s == 0) reinterpret_cast<float*>(chunk + 2 * ACT_PLANE)[tok * 8 + w] = sum;
        if (over) atomicCAS(err, 0, DEV_ERR_OVERFLOW);
        if (seg == 0) {  // zero the 8 padding halfs of both planes
            *reinterpret_cast<uint4*>(chunk + (tok * ACT_ROW_HALFS + 256) * 2) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(chunk + ACT_PLANE + (tok * ACT_ROW_HALFS + 256) * 2) = make_uint4(0, 0, 0, 0);
        }
    } else {
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            uint16_t b[3][4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float f = v[4 * t + e];
#pragma unroll
                for (int pl = 0; pl < 3; ++pl) {
                    const __nv_bfloat16 h = __float2bfloat16_rn(f);
                    b[pl][e] = __bfloat16_as_ushort(h);
                    f -= __bfloat162float(h);
                }
            }
            const int pos = 32 * w + 8 * t + 4 * s;
#pragma unroll
            for (int pl = 0; pl < 3; ++pl) {
                uint2 pk;
                pk.x = (uint32_t)b[pl][0] | ((uint32_t)b[pl][1] << 16);
                pk.y = (uint32_t)b[pl][2] | ((uint32_t)b[pl][3] << 16);
                *reinterpret_cast<uint2*>(chunk + pl * ACT_PLANE + (tok * ACT_ROW_HALFS + pos) * 2) = pk;
            }
        }
        if (seg == 0)
#pragma unroll
            for (int pl = 0; pl < 3; ++pl)
                *reinterpret_cast<uint4*>(chunk + pl * ACT_PLANE + (tok * ACT_ROW_HALFS + 256) * 2) = make_uint4(0, 0, 0, 0);
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

__global__ void reduce_partials_kernel(const float* __restrict__ part, int splits, int n_rows, uint64_t n_out, float* __restrict__ y,
                                       int ld_y) {
    const uint64_t o = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int r = blockIdx.y;
    if (o >= n_out || r >= n_rows) return;
    float v = 0.f;
    for (int s = 0; s < splits; ++s) v += part[((uint64_t)s * MAX_ROWS + r) * n_out + o];
    y[(uint64_t)r * ld_y + o] = v;
}

dfl_status launch_reduce_partials(cudaStream_t st, const float* part, int splits, int n_rows, uint64_t n_out, float* y, int ld_y) {
    dim3 grid((unsigned)((n_out + 255) / 256), (unsigned)n_rows);
    reduce_partials_kernel<<<grid, 256, 0, st>>>(part, splits, n_rows, n_out, y, ld_y);
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
__device__ __forceinline__ Top2 top2_block_reduce(Top2 a) {
    __shared__ Top2 sh[32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Top2 b;
        b.k1 = __shfl_xor_sync(0xffffffffu, a.k1, o);
        b.i1 = __shfl_xor_sync(0xffffffffu, a.i1, o);
        b.k2 = __shfl_xor_sync(0xffffffffu, a.k2, o);
        top2_merge(a, b);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    if (lane == 0) sh[warp] = a;
    __syncthreads();
    if (warp == 0) {
        a = lane < nw ? sh[lane] : Top2{INT32_MIN, INT32_MAX, INT32_MIN, 0};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            Top2 b;
            b.k1 = __shfl_xor_sync(0xffffffffu, a.k1, o);
            b.i1 = __shfl_xor_sync(0xffffffffu, a.i1, o);
            b.k2 = __shfl_xor_sync(0xffffffffu, a.k2, o);
            top2_merge(a, b);
        }
    }
    return a;
}
__device__ __forceinline__ float key_to_float(int32_t k) { return __int_as_float(k < 0 ? (k ^ 0x7fffffff) : k); }

__global__ void argmax_part_kernel(const float* __restrict__ logits, uint64_t vocab, uint64_t ld, Top2* __restrict__ parts) {
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
__global__ void argmax_final_kernel(const Top2* __restrict__ parts, int32_t* __restrict__ argmax, float* __restrict__ gap) {
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
    argmax_part_kernel<<<dim3(ARGMAX_PARTS, n_rows), 256, 0, st>>>(logits, vocab, ld, reinterpret_cast<Top2*>(scratch));
    argmax_final_kernel<<<n_rows, 64, 0, st>>>(reinterpret_cast<const Top2*>(scratch), argmax, gap);
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
