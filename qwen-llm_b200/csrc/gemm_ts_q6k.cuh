// Q6_K for the tensor-memory few-row GEMM: row-lane tile packing, its inverse, and the unpacker.
// Included by gemm_ts.cu only.
//
// A Q6_K weight is d * sc * q with q in [-32, 31] and an int8 scale per 16 columns.  q * sc can
// reach 4096, one bit more than an f16 holds exactly, so the A operand is written as two exact
// matrices that multiply the same activations: A1 = q * (sc & ~1) (even, <= 4096) and
// A2 = q * (sc & 1).
//
// The resident tiles hold the six-bit codes one per BYTE (272 + 2 bytes per 256 weights against ggml's 210).  The
// kernel is bound by the instruction issue of its unpack, not by HBM: with ggml's nibble + 2-bit packing a weight pair
// cost six integer / f16 instructions and the kernel streamed 2.2 TB/s of packed bytes; with byte codes a pair is one
// byte permute under the exponent byte of 1024, one subtract of 1056, one multiply (A1) and one mask (A2), and the 30 %
// more bytes per weight are bytes the memory system had to spare.  The values are ggml's, bit for bit.
//
// Stage (128 rows x 256 columns): [row 128][16 x i8 scales] [row 128][f16 d] [block 8][half 2][row 128][16 bytes], byte j
// of a 32-column block's 32 = the code of the column at position k' = j of the shared activation order (ts_act_kpos).
// Thread (row, kp2) of half h owns block 4 (h / 2) + 2 (h % 2) + kp2, i.e. scale groups 2 block and 2 block + 1.
#pragma once

namespace dfl {

// one thread per (row, 32-column block)
__global__ void retile_ts_q6k_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, uint64_t n_out, int kblocks, int kb_group) {
    const uint64_t tile_id = blockIdx.x;
    const int kb = (int)(tile_id % kblocks);
    const uint64_t rt = tile_id / kblocks;
    uint8_t* stage = dst + tile_id * STAGE_Q6_K_TS;
    for (int idx = threadIdx.x; idx < TILE_R * 8; idx += blockDim.x) {
        const int r = idx & 127, b = idx >> 7;
        const uint64_t row = rt * TILE_R + r;
        const bool valid = row < n_out;
        const uint8_t* blk = src + src_block_index(row, kb, kblocks, n_out, kb_group) * 210ull;
        uint32_t w[8];
#pragma unroll
        for (int wi = 0; wi < 8; ++wi) {
            w[wi] = 0x20202020u;   // code 32 decodes to 0 with any scale
            if (valid) {
                w[wi] = 0u;
#pragma unroll
                for (int j = 0; j < 4; ++j) w[wi] |= q6k_src_q(blk, 32 * b + ts_act_kpos(4 * wi + j)) << (8 * j);   // the order is its own inverse
            }
        }
        uint4* q = reinterpret_cast<uint4*>(stage + TSQ6_OFF_QS);
        q[(b * 2 + 0) * 128 + r] = make_uint4(w[0], w[1], w[2], w[3]);
        q[(b * 2 + 1) * 128 + r] = make_uint4(w[4], w[5], w[6], w[7]);
        if (b == 0) {
            for (int j = 0; j < 16; ++j) stage[r * 16 + j] = valid ? blk[192 + j] : 0;
            reinterpret_cast<uint16_t*>(stage + TSQ6_OFF_D)[r] = valid ? (uint16_t)(blk[208] | (blk[209] << 8)) : 0;
        }
    }
}

__device__ float decode_ts_q6k_elem(const uint8_t* stage, int r, int k) {
    const int b = k >> 5, kprime = ts_act_kpos(k & 31);
    const uint32_t q = stage[TSQ6_OFF_QS + ((b * 2 + (kprime >> 4)) * 128 + r) * 16 + (kprime & 15)];
    const int8_t sc = (int8_t)stage[r * 16 + (k >> 4)];
    const float d = __half2float(__ushort_as_half(reinterpret_cast<const uint16_t*>(stage + TSQ6_OFF_D)[r]));
    return __fmul_rn(__fmul_rn(d, (float)sc), (float)((int)q - 32));
}

namespace ts {

constexpr uint32_t H2_1056 = 0x64206420u;   // half2(1056) = 1024 + 32

template <>
struct Fmt<DFL_Q6_K> {
    static constexpr int STAGE = STAGE_Q6_K_TS;
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
    // r[0..15] = A1 (q * even part of the scale), r[16..31] = A2 (q * odd bit), column c = k' pair (2c, 2c + 1)
    __device__ static __forceinline__ void unpack(const uint8_t* st, int h, int row, int kp2, uint32_t (&r)[32], uint32_t (&)[8],
                                                  UnitScales& us) {
        const int b = 4 * (h >> 1) + 2 * (h & 1) + kp2;
        const uint4* q = reinterpret_cast<const uint4*>(st + TSQ6_OFF_QS);
        const uint4 qa = q[(b * 2 + 0) * 128 + row], qb = q[(b * 2 + 1) * 128 + row];
        us.d = __half2float(__ushort_as_half(reinterpret_cast<const uint16_t*>(st + TSQ6_OFF_D)[row]));
        us.dmin = 0.f;
        const uint32_t sc2 = reinterpret_cast<const uint16_t*>(st)[row * 8 + b];   // int8 scales of groups 2 b, 2 b + 1
        uint32_t se[2], odd[2];
#pragma unroll
        for (int g = 0; g < 2; ++g) {
            const int sc = (int)(int8_t)((sc2 >> (8 * g)) & 0xffu);
            const __half2 e2 = __half2half2(__int2half_rn(sc & ~1));
            se[g] = *reinterpret_cast<const uint32_t*>(&e2);
            odd[g] = (sc & 1) ? 0xffffffffu : 0u;
        }
        const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
#pragma unroll
        for (int wi = 0; wi < 8; ++wi) {
            const int g = wi >> 2;
#pragma unroll
            for (int p = 0; p < 2; ++p) {
                // bytes 2p, 2p + 1 of the word under the exponent byte of 1024: half2(1024 + c0, 1024 + c1), minus 1056 = (q0, q1)
                const uint32_t qq = h2sub(__byte_perm(w[wi], 0x64646464u, p ? 0x4342 : 0x4140), H2_1056);
                r[2 * wi + p] = h2mul(qq, se[g]);
                r[16 + 2 * wi + p] = qq & odd[g];
            }
        }
    }
};

}  // namespace ts
}  // namespace dfl
