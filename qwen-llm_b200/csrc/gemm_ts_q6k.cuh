// Q6_K for the tensor-memory few-row GEMM: row-lane tile packing, its inverse, and the unpacker.
// Included by gemm_ts.cu only.
//
// A Q6_K weight is d * sc * q with q in [-32, 31] and an int8 scale per 16 columns.  q * sc can
// reach 4096, one bit more than an f16 holds exactly, so the A operand is written as two exact
// matrices that multiply the same activations: A1 = q * (sc & ~1) (even, <= 4096) and
// A2 = q * (sc & 1).  A stage is two units of 128 columns; thread (row, kp) owns the 32 columns
// 128 u + 32 kp + l of unit u, i.e. scale groups 8 u + 2 kp and 8 u + 2 kp + 1.
//
// Packing of those 32 six-bit values (k' = position in the shared activation order, see
// ts_act_kpos): four 32-bit words of low nibbles, word wi holding k' = 8 wi .. 8 wi + 7 in the
// nibble order {0, 2, 4, 6, 1, 3, 5, 7} so that four masks of (word shifted by 4, 0, -4, -8) give
// f16 pairs of neighbouring k'; and two 32-bit words of the 2-bit high parts placed so that one
// shift lines them up with bits 8-9 / 24-25 of those pairs.
#pragma once

namespace dfl {

__host__ __device__ inline int tsq6_kprime_of_slot(int wi, int slot) { return 8 * wi + (slot < 4 ? 2 * slot : 2 * (slot - 4) + 1); }
__host__ __device__ inline int tsq6_slot_of_kprime(int within8) { return (within8 & 1) ? 4 + (within8 >> 1) : (within8 >> 1); }
__host__ __device__ inline int tsq6_hi2_bit(int wi, int slot) { return (wi & 1) * 8 + 2 * (slot & 3) + 16 * (slot >> 2); }

// one thread per (row, unit, kp)
__global__ void retile_ts_q6k_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, uint64_t n_out, int kblocks, int kb_group) {
    const uint64_t tile_id = blockIdx.x;
    const int kb = (int)(tile_id % kblocks);
    const uint64_t rt = tile_id / kblocks;
    uint8_t* stage = dst + tile_id * STAGE_Q6_K;
    for (int idx = threadIdx.x; idx < TILE_R * 8; idx += blockDim.x) {
        const int r = idx & 127, kp = (idx >> 7) & 3, u = idx >> 9;
        const uint64_t row = rt * TILE_R + r;
        const bool valid = row < n_out;
        const uint8_t* blk = src + src_block_index(row, kb, kblocks, n_out, kb_group) * 210ull;
        uint32_t nib[4] = {0, 0, 0, 0}, hi2[2] = {0, 0};
        if (valid) {
#pragma unroll
            for (int wi = 0; wi < 4; ++wi)
#pragma unroll
                for (int slot = 0; slot < 8; ++slot) {
                    const int kprime = tsq6_kprime_of_slot(wi, slot);
                    const int l = (kprime & ~3) + (((kprime & 1) << 1) | ((kprime >> 1) & 1));   // the order is its own inverse
                    const uint32_t v = q6k_src_q(blk, 128 * u + 32 * kp + l);
                    nib[wi] |= (v & 15u) << (4 * slot);
                    hi2[wi >> 1] |= (v >> 4) << tsq6_hi2_bit(wi, slot);
                }
        }
        *reinterpret_cast<uint4*>(stage + TSQ6_OFF_NIB + (((u * 4 + kp) * 128) + r) * 16) = make_uint4(nib[0], nib[1], nib[2], nib[3]);
        *reinterpret_cast<uint2*>(stage + TSQ6_OFF_HI2 + (((u * 4 + kp) * 128) + r) * 8) = make_uint2(hi2[0], hi2[1]);
        if (u == 0 && kp == 0) {
            for (int j = 0; j < 16; ++j) stage[r * 16 + j] = valid ? blk[192 + j] : 0;
            reinterpret_cast<uint16_t*>(stage + TSQ6_OFF_D)[r] = valid ? (uint16_t)(blk[208] | (blk[209] << 8)) : 0;
        }
    }
}

__device__ float decode_ts_q6k_elem(const uint8_t* stage, int r, int k) {
    const int u = k >> 7, kp = (k >> 5) & 3, l = k & 31;
    const int kprime = ts_act_kpos(l);
    const int wi = kprime >> 3, slot = tsq6_slot_of_kprime(kprime & 7);
    const uint32_t word = reinterpret_cast<const uint32_t*>(stage + TSQ6_OFF_NIB + (((u * 4 + kp) * 128) + r) * 16)[wi];
    const uint32_t hw = reinterpret_cast<const uint32_t*>(stage + TSQ6_OFF_HI2 + (((u * 4 + kp) * 128) + r) * 8)[wi >> 1];
    const uint32_t q = ((word >> (4 * slot)) & 15u) | (((hw >> tsq6_hi2_bit(wi, slot)) & 3u) << 4);
    const int8_t sc = (int8_t)stage[r * 16 + (k >> 4)];
    const float d = __half2float(__ushort_as_half(reinterpret_cast<const uint16_t*>(stage + TSQ6_OFF_D)[r]));
    return __fmul_rn(__fmul_rn(d, (float)sc), (float)((int)q - 32));
}

namespace ts {

constexpr uint32_t H2_NEG96 = 0xd600d600u;   // half2(-96)

template <>
struct Fmt<DFL_Q6_K> {
    static constexpr int STAGE = STAGE_Q6_K;
    static constexpr int STAGES = KC == 4 ? 5 : 4;
    static constexpr int HALVES = 4;   // half h: unit h / 2 (128 columns), column quarters 2 (h % 2) + kp2; written as A1 (64 columns) and A2 (64)
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
        const int unit = h >> 1, kp = 2 * (h & 1) + kp2;   // columns 128 unit + 32 kp + l of the block
        const uint4 nib = reinterpret_cast<const uint4*>(st + TSQ6_OFF_NIB)[(unit * 4 + kp) * 128 + row];
        const uint2 hi2 = reinterpret_cast<const uint2*>(st + TSQ6_OFF_HI2)[(unit * 4 + kp) * 128 + row];
        us.d = __half2float(__ushort_as_half(reinterpret_cast<const uint16_t*>(st + TSQ6_OFF_D)[row]));
        us.dmin = 0.f;
        const uint32_t sc2 = reinterpret_cast<const uint16_t*>(st)[row * 8 + unit * 4 + kp];   // int8 scales of groups g0, g0 + 1
        uint32_t c1[2], c2[2], c3[2], c4[2];
#pragma unroll
        for (int g = 0; g < 2; ++g) {
            const int sc = (int)(int8_t)((sc2 >> (8 * g)) & 0xffu);
            const __half2 se = __half2half2(__int2half_rn(sc & ~1));
            const uint32_t seb = *reinterpret_cast<const uint32_t*>(&se);
            c1[g] = h2mul(seb, H2_16TH);          // (1024 + 16 v) * se / 16 - 96 se = (v - 32) * se
            c2[g] = h2mul(seb, H2_NEG96);
            c3[g] = (sc & 1) ? H2_16TH : 0u;      // the same with the odd bit as the scale
            c4[g] = (sc & 1) ? H2_NEG96 : 0u;
        }
        const uint32_t w[4] = {nib.x, nib.y, nib.z, nib.w};
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) {
            const uint32_t v = w[wi], hw = wi < 2 ? hi2.x : hi2.y;
            uint32_t x[4];
            if ((wi & 1) == 0) {
                x[0] = ((v << 4) & 0x00f000f0u) | ((hw << 8) & 0x03000300u);
                x[1] = (v & 0x00f000f0u) | ((hw << 6) & 0x03000300u);
                x[2] = ((v >> 4) & 0x00f000f0u) | ((hw << 4) & 0x03000300u);
                x[3] = ((v >> 8) & 0x00f000f0u) | ((hw << 2) & 0x03000300u);
            } else {
                x[0] = ((v << 4) & 0x00f000f0u) | (hw & 0x03000300u);
                x[1] = (v & 0x00f000f0u) | ((hw >> 2) & 0x03000300u);
                x[2] = ((v >> 4) & 0x00f000f0u) | ((hw >> 4) & 0x03000300u);
                x[3] = ((v >> 8) & 0x00f000f0u) | ((hw >> 6) & 0x03000300u);
            }
            const int g = wi >> 1;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                r[4 * wi + q] = h2fma(x[q] | MAGIC, c1[g], c2[g]);
                r[16 + 4 * wi + q] = h2fma(x[q] | MAGIC, c3[g], c4[g]);
            }
        }
    }
};

}  // namespace ts
}  // namespace dfl
