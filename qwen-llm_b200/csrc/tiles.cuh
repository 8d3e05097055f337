// Resident weight layout ("stream tiles") and packed activation layout of the few-row GEMM.
//
// A quantised matrix W[n_out][n_in] arrives in ggml block order
// (crates/qwen-llm/src/tensor.rs:159).  At load it is re-tiled once on the GPU
// (the reference keeps the same "re-pack on load" seam, crates/qwen-llm/src/codec.rs:11-12)
// into tiles of 128 rows x 256 columns, stored [row_tile][k_block][stage bytes], so that
//   * the bytes one CTA needs for one pipeline stage are one contiguous, 16-byte aligned
//     run (a single bulk copy),
//   * each lane of the consuming warp finds the quants of its MMA fragment in one
//     conflict-free 128-bit shared-memory load.
// The total size is unchanged (144 / 176 / 210 / 34 / 2 bytes per block stay what they
// are) and every stored integer keeps its value: only positions move.
//
// Fragment ownership inside a tile.  Warp w (0..7) owns columns [32w, 32w+32) of the
// 256-column block; MMA step s (0,1) covers [32w+16s, +16); lane (g = lane/4, t = lane%4)
// holds, for rows g and g+8 of each 16-row m-tile, the four columns
//   k = 32w + 16s + 4t + e,  e = 0..3,
// with (e0,e1) in the MMA k-slots (2t,2t+1) and (e2,e3) in (2t+8,2t+9).  The activation
// planes use the matching order p(k) = 32w + 8t + 4s + e.
#pragma once
#include <cstdint>

#include "common.cuh"

namespace dfl {

constexpr int TILE_R = 128;   // weight rows per tile
constexpr int TILE_K = 256;   // columns per pipeline stage (one K-quant super-block)
constexpr int MAX_ROWS = 16;  // activation rows (tokens) per GEMM

// stage sizes in bytes = 128 rows x bytes per 256 weights
constexpr int STAGE_Q4_K = TILE_R * 144;  // 18432
constexpr int STAGE_Q5_K = TILE_R * 176;  // 22528
constexpr int STAGE_Q6_K = TILE_R * 210;  // 26880
constexpr int STAGE_Q8_0 = TILE_R * 272;  // 34816
constexpr int STAGE_B16 = TILE_R * 512;   // 65536 (bf16 / f16)

// Q4_K stage: [128 x 16 B header {d,dmin,scales[12]}][quants u32 [w][mt/2][lane][mt%2][rowhalf]]
constexpr int Q4K_OFF_QS = 2048;
// Q5_K stage: header, nibbles as Q4_K, then high bits u8 [w][mt/2][lane][mt%2][rowhalf]
constexpr int Q5K_OFF_QS = 2048;
constexpr int Q5K_OFF_QH = 2048 + 16384;
// Q6_K stage: [128 x 16 i8 scales][128 x f16 d][low nibbles as Q4_K][high 2-bit u16 [w][mt/2][lane][mt%2][rowhalf]]
constexpr int Q6K_OFF_D = 2048;
constexpr int Q6K_OFF_QL = 2304;
constexpr int Q6K_OFF_QH = 2304 + 16384;
// Q8_0 stage: [128 x 8 f16 d][bytes (q ^ 0x80) as u32 [w][mt][lane][rowhalf][step]]
constexpr int Q80_OFF_QS = 2048;
// B16 stage: halfs [w][mt][rowhalf][lane][8] ([step][e])

// Packed activations, one chunk per 256 columns.  f16 variant: hi plane, lo plane
// (x = hi + lo), then the per-32-column sums S[token][8] the K-quant "min" term needs.
// Plane rows are padded to 264 halfs so that the 8 token rows hit different banks.
constexpr int ACT_ROW_HALFS = 264;
constexpr int ACT_PLANE = MAX_ROWS * ACT_ROW_HALFS * 2;  // 8448
constexpr int ACT16_CHUNK = 2 * ACT_PLANE + MAX_ROWS * 8 * 4;  // 17408
// bf16 variant: three planes x = b1 + b2 + b3 (24 significant bits)
constexpr int ACTB3_CHUNK = 3 * ACT_PLANE;  // 25344

__host__ __device__ inline int stage_bytes_of(int dtype) {
    switch (dtype) {
        case DFL_Q4_K: return STAGE_Q4_K;
        case DFL_Q5_K: return STAGE_Q5_K;
        case DFL_Q6_K: return STAGE_Q6_K;
        case DFL_Q8_0: return STAGE_Q8_0;
        case DFL_BF16: return STAGE_B16;
        case DFL_F16: return STAGE_B16;
        default: return 0;
    }
}
// bytes of one ggml row segment of 256 weights
__host__ __device__ inline int ggml_bytes_per_256(int dtype) {
    switch (dtype) {
        case DFL_Q4_K: return 144;
        case DFL_Q5_K: return 176;
        case DFL_Q6_K: return 210;
        case DFL_Q8_0: return 272;
        case DFL_BF16: return 512;
        case DFL_F16: return 512;
        case DFL_F32: return 1024;
        default: return 0;
    }
}
__host__ __device__ inline bool dtype_uses_bf16_acts(int dtype) { return dtype == DFL_BF16; }

// Two resident tile layouts / kernels: per-lane MMA fragments for the mma.sync kernel (this file),
// row-lane tiles for the tensor-memory kernel (gemm_ts.cuh).  The packed activation format
// follows the kernel that consumes it.
constexpr int LAYOUT_FRAG = 0, LAYOUT_TS = 1;
// Q6_K row-lane tiles hold one code per byte: [128 x 16 i8 scales][128 x f16 d][128 rows x 256 bytes]
constexpr int STAGE_Q6_K_TS = 2304 + TILE_R * 256;  // 35072
__host__ __device__ inline int stage_bytes_of(int dtype, int layout) {
    return (dtype == DFL_Q6_K && layout == LAYOUT_TS) ? STAGE_Q6_K_TS : stage_bytes_of(dtype);
}
constexpr int ACT_F16 = 0, ACT_BF3 = 1, ACT_TS = 2, ACT_TSB = 3;
constexpr int ACTTS_CHUNK = 16384 + 1536;  // tensor-memory kernel: B operand + min-term operand per 256 columns
constexpr int ACTTSB_CHUNK = 32 * 768;     // bf16-weight tensor-core kernel: three bf16 planes as one 48-row B operand

// position of column k (0..255) inside an activation plane row
__host__ __device__ inline int act_pos(int k) {
    const int w = k >> 5, s = (k >> 4) & 1, t = (k >> 2) & 3, e = k & 3;
    return 32 * w + 8 * t + 4 * s + e;
}

#ifdef __CUDACC__
// ---- integer quant of weight i (0..255) of one ggml block -------------------
// Q4_K block: {f16 d, f16 dmin, u8 scales[12], u8 qs[128]}  (kernels/mat_vec_q4_k.metal:13-20)
__device__ __forceinline__ uint32_t q4k_src_q(const uint8_t* blk, int i) {
    const int c = i >> 6, l = i & 31, hi = (i >> 5) & 1;
    const uint8_t b = blk[16 + 32 * c + l];
    return hi ? (b >> 4) : (b & 15);
}
// Q5_K block: {d, dmin, scales[12], qh[32], qs[128]}  (kernels/mat_mat_fewrow_gen.metal:72-106)
__device__ __forceinline__ uint32_t q5k_src_q(const uint8_t* blk, int i) {
    const int c = i >> 6, l = i & 31, hi = (i >> 5) & 1;
    const uint8_t b = blk[48 + 32 * c + l];
    const uint32_t nib = hi ? (b >> 4) : (b & 15);
    const uint32_t hb = (blk[16 + l] >> (2 * c + hi)) & 1;
    return nib | (hb << 4);
}
// Q6_K block: {ql[128], qh[64], i8 scales[16], f16 d}  (kernels/mat_vec_q6_k.metal:5-12)
__device__ __forceinline__ uint32_t q6k_src_q(const uint8_t* blk, int i) {
    const int n = i >> 7, rem = i & 127, quarter = rem >> 5, l = rem & 31;
    const uint8_t qlb = blk[64 * n + l + ((quarter & 1) ? 32 : 0)];
    const uint32_t nib = quarter >= 2 ? (qlb >> 4) : (qlb & 15);
    const uint32_t h2 = (blk[128 + 32 * n + l] >> (2 * quarter)) & 3;
    return nib | (h2 << 4);
}

__device__ __forceinline__ void k4_scale_min(const uint8_t* q, int j, uint32_t& sc, uint32_t& m) {
    if (j < 4) { sc = q[j] & 63; m = q[j + 4] & 63; }
    else { sc = (q[j + 4] & 0x0f) | ((q[j - 4] >> 6) << 4); m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
}

// Decoded f32 value of element k (0..255) of one ggml block segment, ggml operation order
// (kernels/mat_vec_q4_k.metal:13-20, mat_vec_q6_k.metal:5-12, mat_vec_q8_0.metal:3-9).
__device__ __forceinline__ float ggml_decode_elem(int dtype, const uint8_t* seg256, int k) {
    switch (dtype) {
        case DFL_Q4_K:
        case DFL_Q5_K: {
            const float d = __half2float(__ushort_as_half((unsigned short)(seg256[0] | (seg256[1] << 8))));
            const float dmin = __half2float(__ushort_as_half((unsigned short)(seg256[2] | (seg256[3] << 8))));
            uint32_t sc, m;
            k4_scale_min(seg256 + 4, k >> 5, sc, m);
            const uint32_t q = dtype == DFL_Q4_K ? q4k_src_q(seg256, k) : q5k_src_q(seg256, k);
            return __fsub_rn(__fmul_rn(d * (float)sc, (float)q), dmin * (float)m);
        }
        case DFL_Q6_K: {
            const float d = __half2float(__ushort_as_half((unsigned short)(seg256[208] | (seg256[209] << 8))));
            const int8_t sc = (int8_t)seg256[192 + (k >> 4)];
            return __fmul_rn(__fmul_rn(d, (float)sc), (float)((int)q6k_src_q(seg256, k) - 32));
        }
        case DFL_Q8_0: {
            const uint8_t* b = seg256 + 34 * (k >> 5);
            const float d = __half2float(__ushort_as_half((unsigned short)(b[0] | (b[1] << 8))));
            return __fmul_rn((float)(int8_t)b[2 + (k & 31)], d);
        }
        case DFL_BF16: return __uint_as_float(((uint32_t)seg256[2 * k] | ((uint32_t)seg256[2 * k + 1] << 8)) << 16);
        case DFL_F16: return __half2float(__ushort_as_half((unsigned short)(seg256[2 * k] | (seg256[2 * k + 1] << 8))));
        case DFL_F32: return reinterpret_cast<const float*>(seg256)[k];
        default: return 0.f;
    }
}
#endif  // __CUDACC__

// A resident matrix.
struct QMatrix {
    int device = 0;
    int dtype = 0;
    int layout = LAYOUT_FRAG;
    uint64_t n_in = 0, n_out = 0;
    int kblocks = 0;    // n_in / 256
    int row_tiles = 0;  // ceil(n_out / 128)
    uint8_t* tiles = nullptr;  // device, [row_tiles][kblocks][stage bytes]; f32 matrices: plain [n_out][n_in]
    bool owns = true;
    uint64_t bytes() const { return (uint64_t)row_tiles * kblocks * stage_bytes_of(dtype, layout); }   // resident bytes: set layout first
    // bytes of the ggml source (what a roofline should count)
    uint64_t ggml_bytes() const { return n_out * (uint64_t)kblocks * ggml_bytes_per_256(dtype); }
};

// ---- host API (tiles.cu / gemm_fewrow.cu) ----------------------------------
// Re-tile a ggml matrix that already sits in device memory.  dst must hold m.bytes().
dfl_status retile_matrix(cudaStream_t st, int dtype, const uint8_t* ggml_dev, uint64_t n_in, uint64_t n_out,
                         uint8_t* dst_tiles);
// Decode resident tiles to f32 [n_out][n_in] (device).
dfl_status decode_tiles(cudaStream_t st, const QMatrix& m, float* out_dev);

// How a GEMM output is scaled per token: y = acc * out_scale * rs[tok], with
// rs = 1/sqrt(sum(partials)/norm_k + eps) when sumsq != nullptr (a fused RMSNorm whose
// element-wise weight was folded into the activations), else 1.
struct GemmEpilogue {
    const float* sumsq = nullptr;  // [n_sumsq][16]
    int n_sumsq = 0;
    float norm_k = 1.f;
    float eps = 0.f;
    float out_scale = 1.f;
    // optional list of row tiles to compute (tensor-memory family only): the kernel works on tiles
    // tile_map[0 .. *n_tiles) of the matrix instead of all of them; both live in device memory and may be
    // written by the preceding kernel.  *n_tiles must be at least the launch's CTAs per split.
    const int32_t* tile_map = nullptr;
    const int32_t* n_tiles = nullptr;
    // the same for the column blocks summed over: blocks kb_map[0 .. *n_kb), *n_kb at least the split count and at most
    // what the splits were chosen for (the activations of a listed block are used as they are)
    const int32_t* kb_map = nullptr;
    const int32_t* n_kb = nullptr;
    // n_kb[1] / n_kb[2] (when n_kb[1] > 0): split count and CTAs per split to use for this list length, their product
    // at most 148, the splits at most the launch's own; the caller sums that many partial slices
    bool dynamic_splits = false;
};
int gemm_choose_splits(const QMatrix& m);
int gemm_max_kblocks_per_cta(int dtype);  // column blocks one CTA can keep resident
// out: [splits][16][n_out] f32 partial sums (sum over the first axis in order 0..splits-1).
// ld_out: row length of `out` (0 = n_out); a wider buffer lets several matrices with the
// same input write side by side (out then points at this matrix's first column).
dfl_status launch_gemm_fewrow(cudaStream_t st, const QMatrix& m, const uint8_t* acts, float* out, int splits,
                              const GemmEpilogue& ep, int* dev_err, bool pdl, uint32_t ld_out = 0);
// x [n_rows][ld] f32 -> packed activations for a matrix of `dtype`; rows >= n_rows are zero.
// pre_scale multiplies x before the f16 split (a power of two keeps it exact).
dfl_status launch_prep_acts(cudaStream_t st, int weight_dtype, const float* x, int ld, int n_rows, uint64_t k,
                            float pre_scale, uint8_t* acts, int* dev_err);
inline uint64_t acts_bytes(int weight_dtype, uint64_t k) {
    return (k / TILE_K) * (uint64_t)(dtype_uses_bf16_acts(weight_dtype) ? ACTB3_CHUNK : ACT16_CHUNK);
}
inline int act_layout_of(const QMatrix& m) {
    if (m.layout == LAYOUT_TS) return dtype_uses_bf16_acts(m.dtype) ? ACT_TSB : ACT_TS;
    return dtype_uses_bf16_acts(m.dtype) ? ACT_BF3 : ACT_F16;
}
inline int act_chunk_bytes(int act_layout) {
    return act_layout == ACT_TS ? ACTTS_CHUNK : act_layout == ACT_TSB ? ACTTSB_CHUNK : act_layout == ACT_BF3 ? ACTB3_CHUNK : ACT16_CHUNK;
}
inline uint64_t acts_bytes_for(const QMatrix& m) { return (m.n_in / TILE_K) * (uint64_t)act_chunk_bytes(act_layout_of(m)); }
// Packs x for the kernel that will consume matrix m.
dfl_status launch_prep_acts_for(cudaStream_t st, const QMatrix& m, const float* x, int ld, int n_rows, float pre_scale, uint8_t* acts,
                                int* dev_err);
// Sum split-K partials: y[r][o] = sum_s part[s][r][o], r < n_rows.
dfl_status launch_reduce_partials(cudaStream_t st, const float* part, int splits, int n_rows, uint64_t n_out,
                                  float* y, int ld_y, const int32_t* splits_dev = nullptr);   // *splits_dev more slices when given
// Row argmax (lowest index on ties, total order) + gap to the runner-up.
dfl_status launch_argmax_top2(cudaStream_t st, const float* logits, int n_rows, uint64_t vocab, uint64_t ld,
                              int32_t* argmax, float* gap, void* scratch /* >= n_rows*ARGMAX_PARTS*16 B */);
// the head's split-K partial sums reduced into `logits` and ranked in the same pass
dfl_status launch_reduce_argmax_top2(cudaStream_t st, const float* part, int splits, int n_rows, uint64_t vocab, float* logits, uint64_t ld,
                                     int32_t* argmax, float* gap, void* scratch);
constexpr int ARGMAX_PARTS = 64;

}  // namespace dfl
