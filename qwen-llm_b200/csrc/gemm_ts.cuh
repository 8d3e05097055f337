// Layouts of the tensor-memory few-row GEMM (gemm_ts.cu): weights are unpacked by the CUDA cores
// into exact f16 integers, stored into tensor memory as the A operand of tcgen05.mma, and the
// packed activations are the B operand read from shared memory.
//
// Weight tiles ("row-lane" tiles, LAYOUT_TS): still [row_tile][k_block][stage bytes], with the
// ggml byte counts except for Q6_K, ordered so that thread (row, kp) of the unpacking CTA - row = its
// tensor-memory lane, kp = its quarter of the 256 columns - finds its bytes with conflict-free
// 128-bit shared-memory loads:
//   Q4_K: [128 x 16 B header {d, dmin, scales[12]}] [kp 4][half 2][row 128][16 B of qs]
//   Q5_K: as Q4_K, then [half 2][row 128][16 B of qh]
//   Q6_K: [128 x 16 B scales i8] [128 x f16 d] [block 8][half 2][row 128][16 B of six-bit codes, one per byte]
//         (35072 bytes per stage instead of ggml's 26880: see gemm_ts_q6k.cuh)
//   Q8_0: [128 x 8 f16 d] [block 8][half 2][row 128][16 B of q + 128]
//
// Activation chunk per 256 columns (ACT_TS): the canonical K-major, no-swizzle operand layout of
// tcgen05.mma: core matrices of 8 rows (n) x 16 bytes (8 halfs along k), the four n-groups of a
// k-core contiguous (128 B apart), k-cores 512 B apart.  n = 2 * token + plane (plane 0 = f16
// hi, 1 = lo, x = hi + lo).  Column k sits at k-position (k & ~3) + {0, 2, 1, 3}[k & 3], the order
// in which the nibble unpack emits its f16 pairs.  After the 16 KiB main operand comes a second,
// small operand for the K-quant "min" term: S[sub-block j][n2 = 3 * token + plane], the sums of
// the activations over each 32-column sub-block as an exact three-way f16 split, K padded from 8
// to 16 with zeros (the second k-core is never written after the buffer was cleared).
#pragma once
#include <cuda_bf16.h>

#include "tiles.cuh"

namespace dfl {

constexpr int TS_B_BYTES = 16384;
constexpr int TS_BMIN_OFF = TS_B_BYTES;
constexpr int TS_BMIN_BYTES = 1536;  // [k-core 2][n-group 6][8][16 B]
static_assert(ACTTS_CHUNK == TS_B_BYTES + TS_BMIN_BYTES, "activation chunk size");

constexpr int TSQ4_OFF_QS = 2048;
constexpr int TSQ5_OFF_QH = 2048 + 16384;
constexpr int TSQ6_OFF_D = 2048;
constexpr int TSQ6_OFF_QS = 2304;

__host__ __device__ inline int ts_act_kpos(int k) { return (k & ~3) + (((k & 1) << 1) | ((k >> 1) & 1)); }
__host__ __device__ inline int ts_b_offset(int n, int kpos) { return (kpos >> 3) * 512 + (n >> 3) * 128 + (n & 7) * 16 + (kpos & 7) * 2; }
__host__ __device__ inline int ts_bmin_offset(int n2, int j) { return TS_BMIN_OFF + (j >> 3) * 768 + (n2 >> 3) * 128 + (n2 & 7) * 16 + (j & 7) * 2; }

// Q8_0 additionally needs its block scales inside a range (q80_scales_fit_ts)
inline bool ts_supported(int dtype) {
    return dtype == DFL_Q4_K || dtype == DFL_Q5_K || dtype == DFL_Q6_K || dtype == DFL_Q8_0 || dtype == DFL_BF16;
}
// bf16-weight operand (gemm_tsb.cuh): n = 3 * token + plane (x = b1 + b2 + b3), natural column order
__host__ __device__ inline int tsb_b_offset(int n, int k) { return (k >> 3) * 768 + (n >> 3) * 128 + (n & 7) * 16 + (k & 7) * 2; }

#ifdef __CUDACC__
// Four consecutive columns k..k+3 (k % 4 == 0) of one token -> hi / lo operand rows.
__device__ __forceinline__ void pack_quad_ts(uint8_t* chunk, int tok, int k, const float (&v)[4], bool& overflow) {
    uint16_t hi[4], lo[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float f = v[e];
        overflow |= (fabsf(f) >= 65504.f) && (fabsf(f) < INFINITY);
        const __half h = __float2half_rn(f);
        hi[e] = __half_as_ushort(h);
        lo[e] = __half_as_ushort(__float2half_rn(f - __half2float(h)));
    }
    // k-positions k + {0, 2, 1, 3}: stored order is v0, v2, v1, v3
    *reinterpret_cast<uint2*>(chunk + ts_b_offset(2 * tok, k)) =
        make_uint2((uint32_t)hi[0] | ((uint32_t)hi[2] << 16), (uint32_t)hi[1] | ((uint32_t)hi[3] << 16));
    *reinterpret_cast<uint2*>(chunk + ts_b_offset(2 * tok + 1, k)) =
        make_uint2((uint32_t)lo[0] | ((uint32_t)lo[2] << 16), (uint32_t)lo[1] | ((uint32_t)lo[3] << 16));
}
__device__ __forceinline__ void pack_quad_tsb(uint8_t* chunk, int tok, int k, const float (&v)[4]) {
    uint16_t b[3][4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        float f = v[e];
#pragma unroll
        for (int pl = 0; pl < 3; ++pl) {
            const __nv_bfloat16 h = __float2bfloat16_rn(f);
            b[pl][e] = __bfloat16_as_ushort(h);
            f -= __bfloat162float(h);
        }
    }
#pragma unroll
    for (int pl = 0; pl < 3; ++pl)
        *reinterpret_cast<uint2*>(chunk + tsb_b_offset(3 * tok + pl, k)) =
            make_uint2((uint32_t)b[pl][0] | ((uint32_t)b[pl][1] << 16), (uint32_t)b[pl][2] | ((uint32_t)b[pl][3] << 16));
}
// Sum of one token's activations over sub-block j (32 columns) -> three f16 planes.
__device__ __forceinline__ void pack_subsum_ts(uint8_t* chunk, int tok, int j, float sum, bool& overflow) {
    float f = sum;
    overflow |= (fabsf(f) >= 65504.f) && (fabsf(f) < INFINITY);
#pragma unroll
    for (int pl = 0; pl < 3; ++pl) {
        const __half h = __float2half_rn(f);
        *reinterpret_cast<__half*>(chunk + ts_bmin_offset(3 * tok + pl, j)) = h;
        *reinterpret_cast<__half*>(chunk + ts_bmin_offset(3 * tok + pl, j + 8)) = __ushort_as_half((unsigned short)0);  // K padding
        f -= __half2float(h);
    }
}
#endif

dfl_status retile_matrix_ts(cudaStream_t st, int dtype, const uint8_t* ggml_dev, uint64_t n_in, uint64_t n_out, uint8_t* dst_tiles,
                            int kb_group = 0);
dfl_status decode_tiles_ts(cudaStream_t st, const QMatrix& m, float* out_dev);
dfl_status q80_scales_fit_ts(cudaStream_t st, const uint8_t* ggml_dev, uint64_t n_in, uint64_t n_out, bool* fits);
dfl_status launch_prep_acts_ts(cudaStream_t st, const float* x, int ld, int n_rows, uint64_t k, float pre_scale, uint8_t* acts,
                               int* dev_err);
dfl_status launch_gemm_ts(cudaStream_t st, const QMatrix& m, const uint8_t* acts, float* out, int splits, const GemmEpilogue& ep,
                          int* dev_err, bool pdl, uint32_t ld_out);
int gemm_ts_choose_splits(const QMatrix& m);
int gemm_ts_choose_splits_multi(const int* row_tiles, int n_mats, int kblocks);
int gemm_ts_ctas_per_split(int row_tiles, int splits);
int gemm_ts_kc();
int gemm_tsb_choose_splits_multi(const int* row_tiles, int n_mats, int kblocks);
dfl_status launch_gemm_tsb(cudaStream_t st, const QMatrix& m, const uint8_t* acts, float* out, int splits, const GemmEpilogue& ep,
                           int* dev_err, bool pdl, uint32_t ld_out);
dfl_status launch_prep_acts_tsb(cudaStream_t st, const float* x, int ld, int n_rows, uint64_t k, float pre_scale, uint8_t* acts);

}  // namespace dfl
