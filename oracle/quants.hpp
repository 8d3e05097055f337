// TEST INFRASTRUCTURE — CPU oracle, never linked into or called by the product.
//
// Scalar restatement of the dequantisation the reference reaches through
// `ggml_get_type_traits(t).to_float` (crates/qwen-llm/src/codec.rs:148-249).  That code
// lives in a third-party dependency that is not vendored in the reference tree:
// llama-cpp-sys-2 0.1.139 (git brittlewis12/llama-cpp-rs rev 4460cc71...,
// Cargo.toml:66, Cargo.lock:1401-1403).  The block formats and loop order below
// restate ggml's published `dequantize_row_*` algorithms and are pinned by the
// reference's own known-answer tests (codec.rs:474-577 for Q8_0 / Q4_K,
// crates/qwen-llm/src/metal/tests/q6_k_f32_tile.rs:27-71 for Q6_K) plus the `gguf`
// Python package's numpy dequantisers for Q5_K / Q6_K.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <vector>

namespace oracle {

enum DType : int32_t { F32 = 0, F16 = 1, Q8_0 = 8, Q4_K = 12, Q5_K = 13, Q6_K = 14, BF16 = 30 };

// (elements per block, bytes per block) — tensor.rs:159 `storage_layout`.
inline void storage_layout(int32_t dt, uint64_t& blk, uint64_t& bytes) {
    switch (dt) {
        case F32: blk = 1; bytes = 4; return;
        case F16: blk = 1; bytes = 2; return;
        case BF16: blk = 1; bytes = 2; return;
        case Q8_0: blk = 32; bytes = 34; return;
        case Q4_K: blk = 256; bytes = 144; return;
        case Q5_K: blk = 256; bytes = 176; return;
        case Q6_K: blk = 256; bytes = 210; return;
        default: throw std::runtime_error("oracle: unsupported dtype");
    }
}

// IEEE binary16 -> binary32, exact (the reference uses the `half` crate).
inline float f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1f;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {  // subnormal: normalise
            int e = -1;
            do { man <<= 1; ++e; } while ((man & 0x400u) == 0);
            man &= 0x3ffu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

// binary32 -> binary16, round to nearest even.
inline uint16_t f32_to_f16(float f) {
    uint32_t x;
    std::memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    int32_t exp = (int32_t)((x >> 23) & 0xff) - 127 + 15;
    uint32_t man = x & 0x7fffffu;
    if (((x >> 23) & 0xff) == 0xff) return (uint16_t)(sign | 0x7c00u | (man ? 0x200u : 0));
    if (exp >= 31) return (uint16_t)(sign | 0x7c00u);
    if (exp <= 0) {
        if (exp < -10) return (uint16_t)sign;
        man |= 0x800000u;
        uint32_t shift = (uint32_t)(14 - exp);
        uint32_t half_man = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half_man & 1))) ++half_man;
        return (uint16_t)(sign | half_man);
    }
    uint32_t half_man = man >> 13;
    uint32_t rem = man & 0x1fffu;
    uint16_t out = (uint16_t)(sign | ((uint32_t)exp << 10) | half_man);
    if (rem > 0x1000u || (rem == 0x1000u && (half_man & 1))) ++out;  // carries into exp correctly
    return out;
}

inline float bf16_to_f32(uint16_t h) {
    uint32_t bits = (uint32_t)h << 16;
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}
inline uint16_t f32_to_bf16(float f) {
    uint32_t x;
    std::memcpy(&x, &f, 4);
    if ((x & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((x >> 16) | 0x40);
    uint32_t lsb = (x >> 16) & 1;
    x += 0x7fffu + lsb;
    return (uint16_t)(x >> 16);
}

inline uint16_t rd16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }

// 6-bit (scale, min) pair j of a K-quant super-block
// (kernels/mat_mat_fewrow_gen.metal:45-69; ggml get_scale_min_k4).
inline void scale_min_k4(int j, const uint8_t* q, uint8_t& sc, uint8_t& m) {
    if (j < 4) {
        sc = q[j] & 63;
        m = q[j + 4] & 63;
    } else {
        sc = (uint8_t)((q[j + 4] & 0x0f) | ((q[j - 4] >> 6) << 4));
        m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

// Q4_K: {f16 d, f16 dmin, u8 scales[12], u8 qs[128]}; value = d*sc*q - dmin*m
// (kernels/mat_vec_q4_k.metal:13-20; pinned by codec.rs:541-577).
inline void dequant_q4_k(const uint8_t* src, float* y, uint64_t n_blocks) {
    for (uint64_t b = 0; b < n_blocks; ++b, src += 144, y += 256) {
        const float d = f16_to_f32(rd16(src));
        const float dmin = f16_to_f32(rd16(src + 2));
        const uint8_t* scales = src + 4;
        const uint8_t* q = src + 16;
        int is = 0;
        float* out = y;
        for (int j = 0; j < 256; j += 64) {
            uint8_t sc, m;
            scale_min_k4(is + 0, scales, sc, m);
            const float d1 = d * sc, m1 = dmin * m;
            scale_min_k4(is + 1, scales, sc, m);
            const float d2 = d * sc, m2 = dmin * m;
            for (int l = 0; l < 32; ++l) *out++ = d1 * (float)(q[l] & 0xf) - m1;
            for (int l = 0; l < 32; ++l) *out++ = d2 * (float)(q[l] >> 4) - m2;
            q += 32;
            is += 2;
        }
    }
}

// Q5_K: {f16 d, f16 dmin, u8 scales[12], u8 qh[32], u8 qs[128]}
// (kernels/mat_mat_fewrow_gen.metal:72-106).
inline void dequant_q5_k(const uint8_t* src, float* y, uint64_t n_blocks) {
    for (uint64_t b = 0; b < n_blocks; ++b, src += 176, y += 256) {
        const float d = f16_to_f32(rd16(src));
        const float dmin = f16_to_f32(rd16(src + 2));
        const uint8_t* scales = src + 4;
        const uint8_t* qh = src + 16;
        const uint8_t* ql = src + 48;
        int is = 0;
        uint8_t u1 = 1, u2 = 2;
        float* out = y;
        for (int j = 0; j < 256; j += 64) {
            uint8_t sc, m;
            scale_min_k4(is + 0, scales, sc, m);
            const float d1 = d * sc, m1 = dmin * m;
            scale_min_k4(is + 1, scales, sc, m);
            const float d2 = d * sc, m2 = dmin * m;
            for (int l = 0; l < 32; ++l)
                *out++ = d1 * (float)((ql[l] & 0xf) + ((qh[l] & u1) ? 16 : 0)) - m1;
            for (int l = 0; l < 32; ++l)
                *out++ = d2 * (float)((ql[l] >> 4) + ((qh[l] & u2) ? 16 : 0)) - m2;
            ql += 32;
            is += 2;
            u1 <<= 2;
            u2 <<= 2;
        }
    }
}

// Q6_K: {u8 ql[128], u8 qh[64], i8 scales[16], f16 d}; value = d*sc*(q-32)
// (kernels/mat_vec_q6_k.metal:5-12; metal/tests/q6_k_f32_tile.rs:27-71).
inline void dequant_q6_k(const uint8_t* src, float* y, uint64_t n_blocks) {
    for (uint64_t b = 0; b < n_blocks; ++b, src += 210, y += 256) {
        const float d = f16_to_f32(rd16(src + 208));
        const uint8_t* ql = src;
        const uint8_t* qh = src + 128;
        const int8_t* sc = (const int8_t*)(src + 192);
        float* out = y;
        for (int n = 0; n < 256; n += 128) {
            for (int l = 0; l < 32; ++l) {
                const int is = l / 16;
                const int8_t q1 = (int8_t)((ql[l + 0] & 0xf) | (((qh[l] >> 0) & 3) << 4)) - 32;
                const int8_t q2 = (int8_t)((ql[l + 32] & 0xf) | (((qh[l] >> 2) & 3) << 4)) - 32;
                const int8_t q3 = (int8_t)((ql[l + 0] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
                const int8_t q4 = (int8_t)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                out[l + 0] = d * sc[is + 0] * q1;
                out[l + 32] = d * sc[is + 2] * q2;
                out[l + 64] = d * sc[is + 4] * q3;
                out[l + 96] = d * sc[is + 6] * q4;
            }
            out += 128;
            ql += 64;
            qh += 32;
            sc += 8;
        }
    }
}

// Q8_0: {f16 d, i8 qs[32]}; value = q*d (kernels/mat_vec_q8_0.metal:3-9;
// pinned by codec.rs:474-538).
inline void dequant_q8_0(const uint8_t* src, float* y, uint64_t n_blocks) {
    for (uint64_t b = 0; b < n_blocks; ++b, src += 34, y += 32) {
        const float d = f16_to_f32(rd16(src));
        const int8_t* q = (const int8_t*)(src + 2);
        for (int l = 0; l < 32; ++l) y[l] = (float)q[l] * d;
    }
}

// codec.rs:287 `dequant_to_f32` for the dtypes on the path.
inline void dequant_to_f32(int32_t dt, const uint8_t* src, uint64_t n_elements, float* y) {
    uint64_t blk, bytes;
    storage_layout(dt, blk, bytes);
    if (n_elements % blk) throw std::runtime_error("oracle: row not block aligned");
    const uint64_t nb = n_elements / blk;
    // Large tensors are decoded in independent runs of blocks on several threads; every value is the same
    // as in one sequential pass (a block never depends on another).
    const int64_t run = 4096, n_runs = (int64_t)((nb + run - 1) / run);
#pragma omp parallel for schedule(static) if (n_runs > 8)
    for (int64_t r = 0; r < n_runs; ++r) {
        const uint64_t b0 = (uint64_t)r * run, n = std::min<uint64_t>(run, nb - b0);
        const uint8_t* s = src + b0 * bytes;
        float* d = y + b0 * blk;
        switch (dt) {
            case F32: std::memcpy(d, s, n * blk * 4); break;
            case F16: for (uint64_t i = 0; i < n * blk; ++i) d[i] = f16_to_f32(rd16(s + 2 * i)); break;
            case BF16: for (uint64_t i = 0; i < n * blk; ++i) d[i] = bf16_to_f32(rd16(s + 2 * i)); break;
            case Q8_0: dequant_q8_0(s, d, n); break;
            case Q4_K: dequant_q4_k(s, d, n); break;
            case Q5_K: dequant_q5_k(s, d, n); break;
            case Q6_K: dequant_q6_k(s, d, n); break;
        }
    }
}

// ---------------------------------------------------------------------------
// Quantisers for synthetic weights.  Only the *decoders* above are pinned to
// ggml; these encoders just have to emit valid blocks (min/max affine fit per
// sub-block), so that oracle and CUDA path decode the same bytes.
// ---------------------------------------------------------------------------
inline void put16(uint8_t* p, uint16_t v) { p[0] = (uint8_t)v; p[1] = (uint8_t)(v >> 8); }
inline int iround(float v) { return (int)lrintf(v); }
inline int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

inline void pack_scales_k4(const uint8_t sc[8], const uint8_t mn[8], uint8_t out[12]) {
    for (int j = 0; j < 4; ++j) {
        out[j] = (uint8_t)((sc[j] & 63) | ((sc[j + 4] >> 4) << 6));
        out[4 + j] = (uint8_t)((mn[j] & 63) | ((mn[j + 4] >> 4) << 6));
        out[8 + j] = (uint8_t)((sc[j + 4] & 0x0f) | ((mn[j + 4] & 0x0f) << 4));
    }
}

inline void quant_k45(const float* x, uint8_t* dst, uint64_t n_blocks, int levels /*15|31*/) {
    const int bytes = levels == 15 ? 144 : 176;
    for (uint64_t b = 0; b < n_blocks; ++b, x += 256, dst += bytes) {
        float scl[8], mns[8], max_s = 0.f, max_m = 0.f;
        for (int j = 0; j < 8; ++j) {
            float lo = x[32 * j], hi = lo;
            for (int l = 1; l < 32; ++l) { lo = std::fmin(lo, x[32 * j + l]); hi = std::fmax(hi, x[32 * j + l]); }
            if (lo > 0.f) lo = 0.f;
            scl[j] = (hi - lo) / (float)levels;
            mns[j] = -lo;
            max_s = std::fmax(max_s, scl[j]);
            max_m = std::fmax(max_m, mns[j]);
        }
        const uint16_t dh = f32_to_f16(max_s / 63.f), mh = f32_to_f16(max_m / 63.f);
        const float d = f16_to_f32(dh), dmin = f16_to_f32(mh);
        uint8_t sc[8], mn[8];
        for (int j = 0; j < 8; ++j) {
            sc[j] = (uint8_t)clampi(d > 0.f ? iround(scl[j] / d) : 0, 0, 63);
            mn[j] = (uint8_t)clampi(dmin > 0.f ? iround(mns[j] / dmin) : 0, 0, 63);
        }
        put16(dst, dh);
        put16(dst + 2, mh);
        pack_scales_k4(sc, mn, dst + 4);
        uint8_t* qh = dst + 16;
        uint8_t* qs = dst + (levels == 15 ? 16 : 48);
        if (levels == 31) std::memset(qh, 0, 32);
        for (int j = 0; j < 8; ++j) {
            const float ds = d * sc[j], dm = dmin * mn[j];
            for (int l = 0; l < 32; ++l) {
                int q = ds > 0.f ? iround((x[32 * j + l] + dm) / ds) : 0;
                q = clampi(q, 0, levels);
                uint8_t* byte = qs + 32 * (j / 2) + l;
                if (j & 1) *byte = (uint8_t)((*byte & 0x0f) | ((q & 15) << 4));
                else *byte = (uint8_t)(q & 15);
                if (levels == 31 && (q & 16)) qh[l] |= (uint8_t)(1u << j);
            }
        }
    }
}

inline void quant_q6_k(const float* x, uint8_t* dst, uint64_t n_blocks) {
    for (uint64_t b = 0; b < n_blocks; ++b, x += 256, dst += 210) {
        float scl[16], max_abs_s = 0.f;
        for (int j = 0; j < 16; ++j) {
            float amax = 0.f;
            for (int l = 0; l < 16; ++l) amax = std::fmax(amax, std::fabs(x[16 * j + l]));
            scl[j] = amax / 31.f;
            max_abs_s = std::fmax(max_abs_s, scl[j]);
        }
        const uint16_t dh = f32_to_f16(max_abs_s / 127.f);
        const float d = f16_to_f32(dh);
        int8_t sc[16];
        uint8_t q[256];
        for (int j = 0; j < 16; ++j) {
            sc[j] = (int8_t)clampi(d > 0.f ? iround(scl[j] / d) : 0, -128, 127);
            const float ds = d * sc[j];
            for (int l = 0; l < 16; ++l)
                q[16 * j + l] = (uint8_t)(clampi(ds != 0.f ? iround(x[16 * j + l] / ds) : 0, -32, 31) + 32);
        }
        uint8_t* ql = dst;
        uint8_t* qh = dst + 128;
        std::memset(dst, 0, 192);
        for (int n = 0; n < 2; ++n) {
            for (int l = 0; l < 32; ++l) {
                const uint8_t q1 = q[128 * n + l], q2 = q[128 * n + 32 + l];
                const uint8_t q3 = q[128 * n + 64 + l], q4 = q[128 * n + 96 + l];
                ql[64 * n + l] = (uint8_t)((q1 & 15) | ((q3 & 15) << 4));
                ql[64 * n + 32 + l] = (uint8_t)((q2 & 15) | ((q4 & 15) << 4));
                qh[32 * n + l] = (uint8_t)((q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6));
            }
        }
        std::memcpy(dst + 192, sc, 16);
        put16(dst + 208, dh);
    }
}

inline void quant_q8_0(const float* x, uint8_t* dst, uint64_t n_blocks) {
    for (uint64_t b = 0; b < n_blocks; ++b, x += 32, dst += 34) {
        float amax = 0.f;
        for (int l = 0; l < 32; ++l) amax = std::fmax(amax, std::fabs(x[l]));
        const uint16_t dh = f32_to_f16(amax / 127.f);
        const float d = f16_to_f32(dh);
        put16(dst, dh);
        for (int l = 0; l < 32; ++l) dst[2 + l] = (uint8_t)(int8_t)clampi(d > 0.f ? iround(x[l] / d) : 0, -127, 127);
    }
}

inline void quantize_from_f32(int32_t dt, const float* x, uint64_t n_elements, uint8_t* dst) {
    uint64_t blk, bytes;
    storage_layout(dt, blk, bytes);
    if (n_elements % blk) throw std::runtime_error("oracle: row not block aligned");
    const uint64_t nb = n_elements / blk;
    switch (dt) {
        case F32: std::memcpy(dst, x, n_elements * 4); return;
        case F16: for (uint64_t i = 0; i < n_elements; ++i) put16(dst + 2 * i, f32_to_f16(x[i])); return;
        case BF16: for (uint64_t i = 0; i < n_elements; ++i) put16(dst + 2 * i, f32_to_bf16(x[i])); return;
        case Q8_0: quant_q8_0(x, dst, nb); return;
        case Q4_K: quant_k45(x, dst, nb, 15); return;
        case Q5_K: quant_k45(x, dst, nb, 31); return;
        case Q6_K: quant_q6_k(x, dst, nb); return;
    }
}

}  // namespace oracle
