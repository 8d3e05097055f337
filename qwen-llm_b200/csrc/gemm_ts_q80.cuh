// Q8_0 for the tensor-memory few-row GEMM: row-lane tile packing, its inverse, and the unpacker.
// Included by gemm_ts.cu only.
//
// A Q8_0 weight is d * q with q an int8 and one f16 scale d per 32 columns, a different one in every row, so the scale
// cannot wait for the read-back as the K-quants' super-block scale does: it is folded into the A operand.  q * d has up
// to 19 significant bits, more than an f16 holds, so the operand is written as two matrices that multiply the same
// activations, A1 = fl16(q * d) and A2 = q * d - A1.  Every f16 is a multiple of 2^-24 and q is an integer, so the
// remainder is a multiple of 2^-24 no larger than half an ulp of A1: it is an f16 (possibly subnormal) and the fused
// multiply-add that forms it returns it exactly.  A1 + A2 == q * d for every finite d with |128 d| below the f16 range,
// which the loader checks (|d| <= 256; other matrices stay on the mma.sync kernel).
//
// Stage (128 rows x 256 columns, the ggml byte count): [row 128][8 x f16 d] [block 8][half 2][row 128][16 bytes], byte j of
// a block's 32 = q + 128 of the column at position k' = j of the shared activation order (ts_act_kpos).  Thread
// (row, kp2) of half h owns block 4 (h / 2) + 2 (h % 2) + kp2: the same column ownership and MMA mapping as Q6_K.
#pragma once

namespace dfl {

constexpr int TSQ8_OFF_QS = 2048;

// one thread per (row, block)
__global__ void retile_ts_q80_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, uint64_t n_out, int kblocks, int kb_group) {
    const uint64_t tile_id = blockIdx.x;
    const int kb = (int)(tile_id % kblocks);
    const uint64_t rt = tile_id / kblocks;
    uint8_t* stage = dst + tile_id * STAGE_Q8_0;
    for (int idx = threadIdx.x; idx < TILE_R * 8; idx += blockDim.x) {
        const int r = idx & 127, b = idx >> 7;
        const uint64_t row = rt * TILE_R + r;
        const bool valid = row < n_out;
        const uint8_t* blk = src + src_block_index(row, kb, kblocks, n_out, kb_group) * 272ull + 34 * b;
        uint32_t w[8];
#pragma unroll
        for (int wi = 0; wi < 8; ++wi) {
            w[wi] = 0x80808080u;   // q = 0
            if (valid) {
                w[wi] = 0u;
#pragma unroll
                for (int j = 0; j < 4; ++j) w[wi] |= (uint32_t)(uint8_t)(blk[2 + ts_act_kpos(4 * wi + j)] ^ 0x80u) << (8 * j);   // the order is its own inverse
            }
        }
        uint4* q = reinterpret_cast<uint4*>(stage + TSQ8_OFF_QS);
        q[(b * 2 + 0) * 128 + r] = make_uint4(w[0], w[1], w[2], w[3]);
        q[(b * 2 + 1) * 128 + r] = make_uint4(w[4], w[5], w[6], w[7]);
        reinterpret_cast<uint16_t*>(stage)[r * 8 + b] = valid ? (uint16_t)(blk[0] | (blk[1] << 8)) : (uint16_t)0;
    }
}

__device__ float decode_ts_q80_elem(const uint8_t* stage, int r, int k) {
    const int b = k >> 5, kprime = ts_act_kpos(k & 31);
    const uint8_t u = stage[TSQ8_OFF_QS + ((b * 2 + (kprime >> 4)) * 128 + r) * 16 + (kprime & 15)];
    const float d = __half2float(__ushort_as_half(reinterpret_cast<const uint16_t*>(stage)[r * 8 + b]));
    return __fmul_rn((float)((int)u - 128), d);
}

// 1 in *flag when a scale of the matrix is not finite or larger than 256 in magnitude (then q * d may leave the f16 range)
__global__ void q80_scale_range_kernel(const uint8_t* __restrict__ src, uint64_t n_blocks, int* flag) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_blocks) return;
    const uint8_t* blk = src + i * 34ull;
    const float d = __half2float(__ushort_as_half((unsigned short)(blk[0] | (blk[1] << 8))));
    if (!(fabsf(d) <= 256.f)) *flag = 1;
}

namespace ts {

constexpr uint32_t H2_1152 = 0x64806480u;   // half2(1152) = 1024 + 128

template <>
struct Fmt<DFL_Q8_0> {
    static constexpr int STAGE = STAGE_Q8_0;
    static constexpr int STAGES = KC == 4 ? 4 : 3;
    static constexpr int HALVES = 4;   // half h: blocks 4 (h / 2) + 2 (h % 2) + kp2; written as A1 (64 columns) and A2 (64)
    static constexpr bool HAS_MIN = false;
    // steps 0..3 multiply A1, steps 4..7 A2, both with the half's four 16-column slices
    __device__ static __forceinline__ uint32_t a_col(int h, int jj) { return (uint32_t)((jj < 4 ? 0 : 64) + 32 * (h & 1) + 8 * (jj & 3)); }
    __device__ static __forceinline__ uint32_t b_slice(int h, int jj) { return (uint32_t)(8 * (h >> 1) + 4 * (h & 1) + (jj & 3)); }
    __device__ static __forceinline__ void store(uint32_t buf, int h, int kp2, const uint32_t (&r)[32]) {
        const int kp = 2 * (h & 1) + kp2;
        uint32_t lo[16], hi[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) { lo[i] = r[i]; hi[i] = r[16 + i]; }
        tmem_st16(buf + 16 * kp, lo);
        tmem_st16(buf + 64 + 16 * kp, hi);
    }
    __device__ static __forceinline__ int min_col(int, int) { return 0; }
    // r[0..15] = A1, r[16..31] = A2, column c = k' pair (2c, 2c + 1)
    __device__ static __forceinline__ void unpack(const uint8_t* st, int h, int row, int kp2, uint32_t (&r)[32], uint32_t (&)[8],
                                                  UnitScales& us) {
        const int b = 4 * (h >> 1) + 2 * (h & 1) + kp2;
        const uint4* q = reinterpret_cast<const uint4*>(st + TSQ8_OFF_QS);
        const uint4 qa = q[(b * 2 + 0) * 128 + row], qb = q[(b * 2 + 1) * 128 + row];
        const uint32_t d1 = reinterpret_cast<const uint16_t*>(st)[row * 8 + b];
        const uint32_t dd = d1 | (d1 << 16);
        us.d = 1.f;
        us.dmin = 0.f;
        const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
#pragma unroll
        for (int wi = 0; wi < 8; ++wi) {
#pragma unroll
            for (int p = 0; p < 2; ++p) {
                // bytes 2p, 2p + 1 of the word under the exponent byte of 1024: half2(1024 + u0, 1024 + u1), minus 1152 = (q0, q1)
                const uint32_t qq = h2sub(__byte_perm(w[wi], 0x64646464u, p ? 0x4342 : 0x4140), H2_1152);
                const uint32_t a1 = h2mul(qq, dd);
                r[2 * wi + p] = a1;
                r[16 + 2 * wi + p] = h2fma(qq, dd, a1 ^ 0x80008000u);
            }
        }
    }
};

}  // namespace ts
}  // namespace dfl
