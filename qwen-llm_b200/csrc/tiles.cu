// Re-tiling of ggml block matrices into the resident stream-tile layout, and the inverse
// decode used to prove that every stored integer kept its value
// (the check the reference makes in crates/qwen-llm/src/metal_dflash/tests.rs:2774-2822 and
// crates/qwen-llm/src/metal/tests/q6_k_f32_tile.rs:96-102).
#include "tiles.cuh"

namespace dfl {

// One thread per (row in tile, warp slot w, lane slot t): the 8 weights
// k = 32w + 16s + 4t + e of one 256-column block.
template <int DT>
__global__ void retile_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, uint64_t n_out, int kblocks,
                              int row_tiles) {
    constexpr int SRC_BLK = DT == DFL_Q4_K ? 144 : DT == DFL_Q5_K ? 176 : DT == DFL_Q6_K ? 210 : DT == DFL_Q8_0 ? 272 : 512;
    constexpr int STAGE = DT == DFL_Q4_K ? STAGE_Q4_K : DT == DFL_Q5_K ? STAGE_Q5_K : DT == DFL_Q6_K ? STAGE_Q6_K
                        : DT == DFL_Q8_0 ? STAGE_Q8_0 : STAGE_B16;
    const uint64_t tile_id = blockIdx.x;  // row_tile * kblocks + kb
    const int kb = (int)(tile_id % kblocks);
    const uint64_t rt = tile_id / kblocks;
    uint8_t* stage = dst + tile_id * STAGE;
    for (int idx = threadIdx.x; idx < TILE_R * 32; idx += blockDim.x) {
        const int r = idx >> 5, w = (idx >> 2) & 7, t = idx & 3;
        const uint64_t row = rt * TILE_R + r;
        const bool valid = row < n_out;
        const uint8_t* blk = src + (row * kblocks + kb) * (uint64_t)SRC_BLK;
        const int mt = r >> 4, g = r & 7, rh = (r >> 3) & 1, lane = g * 4 + t;
        uint32_t q[8];  // [s*4 + e]
#pragma unroll
        for (int s = 0; s < 2; ++s)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int k = 32 * w + 16 * s + 4 * t + e;
                uint32_t v = 0;
                if (valid) {
                    if (DT == DFL_Q4_K) v = q4k_src_q(blk, k);
                    else if (DT == DFL_Q5_K) v = q5k_src_q(blk, k);
                    else if (DT == DFL_Q6_K) v = q6k_src_q(blk, k);
                    else if (DT == DFL_Q8_0) v = blk[34 * (k >> 5) + 2 + (k & 31)];
                    else v = (uint32_t)blk[2 * k] | ((uint32_t)blk[2 * k + 1] << 8);
                } else if (DT == DFL_Q6_K) v = 32;  // decodes to 0 with any scale
                q[s * 4 + e] = v;
            }
        if (DT == DFL_Q4_K || DT == DFL_Q5_K || DT == DFL_Q6_K) {
            // nibble plane: byte (s + 2*(e&1)), nibble (e>>1)
            uint32_t word = 0;
#pragma unroll
            for (int s = 0; s < 2; ++s)
#pragma unroll
                for (int e = 0; e < 4; ++e) word |= (q[s * 4 + e] & 15u) << (8 * (s + 2 * (e & 1)) + 4 * (e >> 1));
            const int off_qs = DT == DFL_Q6_K ? Q6K_OFF_QL : Q4K_OFF_QS;
            uint32_t* qs = reinterpret_cast<uint32_t*>(stage + off_qs);
            qs[(((w * 4 + (mt >> 1)) * 32 + lane) * 2 + (mt & 1)) * 2 + rh] = word;
            if (DT == DFL_Q5_K) {
                uint32_t hb = 0;  // bit 4*(e&1) + 2*s + (e>>1)
#pragma unroll
                for (int s = 0; s < 2; ++s)
#pragma unroll
                    for (int e = 0; e < 4; ++e) hb |= ((q[s * 4 + e] >> 4) & 1u) << (4 * (e & 1) + 2 * s + (e >> 1));
                stage[Q5K_OFF_QH + (((w * 4 + (mt >> 1)) * 32 + lane) * 2 + (mt & 1)) * 2 + rh] = (uint8_t)hb;
            }
            if (DT == DFL_Q6_K) {
                uint32_t hh = 0;  // 2-bit field at 8*(e&1) + 2*(2*s + (e>>1))
#pragma unroll
                for (int s = 0; s < 2; ++s)
#pragma unroll
                    for (int e = 0; e < 4; ++e) hh |= ((q[s * 4 + e] >> 4) & 3u) << (8 * (e & 1) + 2 * (2 * s + (e >> 1)));
                uint16_t* qh = reinterpret_cast<uint16_t*>(stage + Q6K_OFF_QH);
                qh[(((w * 4 + (mt >> 1)) * 32 + lane) * 2 + (mt & 1)) * 2 + rh] = (uint16_t)hh;
            }
        } else if (DT == DFL_Q8_0) {
            uint32_t* qs = reinterpret_cast<uint32_t*>(stage + Q80_OFF_QS);
#pragma unroll
            for (int s = 0; s < 2; ++s) {
                uint32_t word = 0;
#pragma unroll
                for (int e = 0; e < 4; ++e) word |= ((q[s * 4 + e] ^ 0x80u) & 0xffu) << (8 * e);
                qs[(((w * 8 + mt) * 32 + lane) * 2 + rh) * 2 + s] = word;
            }
        } else {  // 16-bit floats
            uint16_t* qs = reinterpret_cast<uint16_t*>(stage);
#pragma unroll
            for (int j = 0; j < 8; ++j) qs[((((w * 8 + mt) * 2 + rh) * 32 + lane) * 8) + j] = (uint16_t)q[j];
        }
        // per-row header fields, written once per row
        if (w == 0 && t == 0) {
            if (DT == DFL_Q4_K || DT == DFL_Q5_K) {
                uint32_t* h = reinterpret_cast<uint32_t*>(stage + r * 16);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint32_t v = 0;
                    if (valid) v = blk[4 * j] | (blk[4 * j + 1] << 8) | (blk[4 * j + 2] << 16) | ((uint32_t)blk[4 * j + 3] << 24);
                    h[j] = v;
                }
            } else if (DT == DFL_Q6_K) {
                for (int j = 0; j < 16; ++j) stage[r * 16 + j] = valid ? blk[192 + j] : 0;
                reinterpret_cast<uint16_t*>(stage + Q6K_OFF_D)[r] = valid ? (uint16_t)(blk[208] | (blk[209] << 8)) : 0;
            } else if (DT == DFL_Q8_0) {
                uint16_t* d = reinterpret_cast<uint16_t*>(stage);
                for (int j = 0; j < 8; ++j) d[r * 8 + j] = valid ? (uint16_t)(blk[34 * j] | (blk[34 * j + 1] << 8)) : 0;
            }
        }
    }
}

dfl_status retile_matrix(cudaStream_t st, int dtype, const uint8_t* ggml_dev, uint64_t n_in, uint64_t n_out,
                         uint8_t* dst_tiles) {
    if (n_in % TILE_K) return fail(DFL_ERR_BAD_SHAPE, "retile: n_in must be a multiple of 256");
    const int kblocks = (int)(n_in / TILE_K);
    const int row_tiles = (int)((n_out + TILE_R - 1) / TILE_R);
    const uint64_t n_tiles = (uint64_t)kblocks * row_tiles;
    if (n_tiles == 0 || n_tiles > 0x7fffffffu) return fail(DFL_ERR_BAD_SHAPE, "retile: tile count out of range");
    dim3 grid((unsigned)n_tiles), block(256);
    switch (dtype) {
        case DFL_Q4_K: retile_kernel<DFL_Q4_K><<<grid, block, 0, st>>>(ggml_dev, dst_tiles, n_out, kblocks, row_tiles); break;
        case DFL_Q5_K: retile_kernel<DFL_Q5_K><<<grid, block, 0, st>>>(ggml_dev, dst_tiles, n_out, kblocks, row_tiles); break;
        case DFL_Q6_K: retile_kernel<DFL_Q6_K><<<grid, block, 0, st>>>(ggml_dev, dst_tiles, n_out, kblocks, row_tiles); break;
        case DFL_Q8_0: retile_kernel<DFL_Q8_0><<<grid, block, 0, st>>>(ggml_dev, dst_tiles, n_out, kblocks, row_tiles); break;
        case DFL_BF16:
        case DFL_F16: retile_kernel<DFL_BF16><<<grid, block, 0, st>>>(ggml_dev, dst_tiles, n_out, kblocks, row_tiles); break;
        default: return fail(DFL_ERR_UNSUPPORTED, "retile: dtype");
    }
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

// ---- decode: resident tiles -> f32, ggml operation order ----------------------
__global__ void decode_tiles_kernel(const uint8_t* __restrict__ tiles, int dtype, uint64_t n_in, uint64_t n_out, int kblocks,
                                    float* __restrict__ out) {
    const uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_in * n_out) return;
    const uint64_t row = idx / n_in;
    const int kk = (int)(idx % n_in);
    const int kb = kk >> 8, k = kk & 255;
    const uint64_t rt = row / TILE_R;
    const int r = (int)(row % TILE_R);
    const uint8_t* stage = tiles + (rt * kblocks + kb) * (uint64_t)stage_bytes_of(dtype);
    const int w = k >> 5, s = (k >> 4) & 1, t = (k >> 2) & 3, e = k & 3;
    const int mt = r >> 4, g = r & 7, rh = (r >> 3) & 1, lane = g * 4 + t;
    const int slot = (((w * 4 + (mt >> 1)) * 32 + lane) * 2 + (mt & 1)) * 2 + rh;
    float v = 0.f;
    if (dtype == DFL_Q4_K || dtype == DFL_Q5_K) {
        const uint8_t* h = stage + r * 16;
        const float d = __half2float(__ushort_as_half((unsigned short)(h[0] | (h[1] << 8))));
        const float dmin = __half2float(__ushort_as_half((unsigned short)(h[2] | (h[3] << 8))));
        uint32_t sc, m;
        k4_scale_min(h + 4, w, sc, m);
        const uint32_t word = reinterpret_cast<const uint32_t*>(stage + Q4K_OFF_QS)[slot];
        uint32_t q = (word >> (8 * (s + 2 * (e & 1)) + 4 * (e >> 1))) & 15u;
        if (dtype == DFL_Q5_K) q |= ((stage[Q5K_OFF_QH + slot] >> (4 * (e & 1) + 2 * s + (e >> 1))) & 1u) << 4;
        const float d1 = d * (float)sc, m1 = dmin * (float)m;
        v = __fsub_rn(__fmul_rn(d1, (float)q), m1);
    } else if (dtype == DFL_Q6_K) {
        const int8_t sc = (int8_t)stage[r * 16 + 2 * w + s];
        const float d = __half2float(__ushort_as_half(reinterpret_cast<const uint16_t*>(stage + Q6K_OFF_D)[r]));
        const uint32_t word = reinterpret_cast<const uint32_t*>(stage + Q6K_OFF_QL)[slot];
        const uint32_t hh = reinterpret_cast<const uint16_t*>(stage + Q6K_OFF_QH)[slot];
        const uint32_t q = ((word >> (8 * (s + 2 * (e & 1)) + 4 * (e >> 1))) & 15u) |
                           (((hh >> (8 * (e & 1) + 2 * (2 * s + (e >> 1)))) & 3u) << 4);
        v = __fmul_rn(__fmul_rn(d, (float)sc), (float)((int)q - 32));
    } else if (dtype == DFL_Q8_0) {
        const float d = __half2float(__ushort_as_half(reinterpret_cast<const uint16_t*>(stage)[r * 8 + w]));
        const uint32_t word = reinterpret_cast<const uint32_t*>(stage + Q80_OFF_QS)[(((w * 8 + mt) * 32 + lane) * 2 + rh) * 2 + s];
        const int q = (int)(int8_t)(((word >> (8 * e)) & 0xffu) ^ 0x80u);
        v = __fmul_rn((float)q, d);
    } else {
        const uint16_t bits = reinterpret_cast<const uint16_t*>(stage)[((((w * 8 + mt) * 2 + rh) * 32 + lane) * 8) + s * 4 + e];
        v = dtype == DFL_BF16 ? __uint_as_float((uint32_t)bits << 16) : __half2float(__ushort_as_half(bits));
    }
    out[idx] = v;
}

dfl_status decode_tiles(cudaStream_t st, const QMatrix& m, float* out_dev) {
    const uint64_t n = m.n_in * m.n_out;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    decode_tiles_kernel<<<blocks, 256, 0, st>>>(m.tiles, m.dtype, m.n_in, m.n_out, m.kblocks, out_dev);
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

}  // namespace dfl
