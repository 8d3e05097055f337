// Element-wise kernels between two GEMMs: split-K reduction, residual add, SwiGLU, folding of
// the RMSNorm weight, hidden-state capture and packing of the next GEMM's activations, in one
// pass.  Replaces the reference's separate kernel_add_inplace_f32 / kernel_silu_mul_f32 /
// kernel_rms_norm_batched_f32 launches (kernels/elementwise.metal:89,193; rms_norm.metal:48).
//
// RMSNorm is split so that no row-wide reduction sits on the critical path: this kernel
// multiplies by the norm weight and emits per-256-column partial sums of squares; the
// consuming GEMM multiplies its result by 1/sqrt(mean(x^2) + eps) per token.
#include "ops.cuh"

namespace dfl {

// grid = k / 256, block 256: thread = (token = tid / 16, 16 consecutive columns).
__global__ void __launch_bounds__(256) glue_kernel(const GlueParams p) {
    const int kb = blockIdx.x, tok = threadIdx.x >> 4, seg = threadIdx.x & 15;
    const int col0 = kb * TILE_K + seg * 16;
    const bool live = tok < p.n_rows;
    float v[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = 0.f;
    if (live) {
        if (p.mode == GLUE_SWIGLU) {
            float g[16], u[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) { g[j] = 0.f; u[j] = 0.f; }
            for (int s = 0; s < p.splits; ++s) {
                const float* base = p.part + ((uint64_t)s * MAX_ROWS + tok) * p.ld_part + col0;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float4 a = reinterpret_cast<const float4*>(base)[j];
                    const float4 b = reinterpret_cast<const float4*>(base + p.swiglu_f)[j];
                    g[4 * j] += a.x; g[4 * j + 1] += a.y; g[4 * j + 2] += a.z; g[4 * j + 3] += a.w;
                    u[4 * j] += b.x; u[4 * j + 1] += b.y; u[4 * j + 2] += b.z; u[4 * j + 3] += b.w;
                }
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = silu_f(g[j]) * u[j];
        } else {
            if (p.x) {
                const float4* src = reinterpret_cast<const float4*>(p.x + (uint64_t)tok * p.ld_x + col0);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float4 a = src[j];
                    v[4 * j] = a.x; v[4 * j + 1] = a.y; v[4 * j + 2] = a.z; v[4 * j + 3] = a.w;
                }
            }
            if (p.mode == GLUE_RESID && p.part) {
                // sum the split-K partials first (fixed order), then add to the residual
                float acc[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[j] = 0.f;
                for (int s = 0; s < p.splits; ++s) {
                    const float4* src = reinterpret_cast<const float4*>(p.part + ((uint64_t)s * MAX_ROWS + tok) * p.ld_part + col0);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float4 a = src[j];
                        acc[4 * j] += a.x; acc[4 * j + 1] += a.y; acc[4 * j + 2] += a.z; acc[4 * j + 3] += a.w;
                    }
                }
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] += acc[j];
                if (p.x) {
                    float4* dst = reinterpret_cast<float4*>(p.x + (uint64_t)tok * p.ld_x + col0);
#pragma unroll
                    for (int j = 0; j < 4; ++j) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                }
            }
        }
        if (p.capture) {
            float4* dst = reinterpret_cast<float4*>(p.capture + (uint64_t)tok * p.ld_capture + col0);
#pragma unroll
            for (int j = 0; j < 4; ++j) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        }
    }
    if (p.sumsq) {
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) ss += v[j] * v[j];
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (seg == 0) p.sumsq[kb * MAX_ROWS + tok] = ss;
    }
    if (p.mul_w) {
        const float4* w = reinterpret_cast<const float4*>(p.mul_w + col0);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float4 a = w[j];
            v[4 * j] *= a.x; v[4 * j + 1] *= a.y; v[4 * j + 2] *= a.z; v[4 * j + 3] *= a.w;
        }
    }
    if (p.pre_scale != 1.f) {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] *= p.pre_scale;
    }
    if (p.xn && live) {
        float4* dst = reinterpret_cast<float4*>(p.xn + (uint64_t)tok * p.ld_xn + col0);
#pragma unroll
        for (int j = 0; j < 4; ++j) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    }
    if (p.acts) {
        uint8_t* chunk = p.acts + (uint64_t)kb * (p.bf3 ? ACTB3_CHUNK : ACT16_CHUNK);
        bool over = false;
        float sum = 0.f;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float quad[4] = {v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]};
            pack_quad(chunk, p.bf3 != 0, tok, seg * 16 + 4 * q, quad, over);
            sum += quad[0] + quad[1] + quad[2] + quad[3];
        }
        if (!p.bf3) {
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);  // 32-column sub-block = two neighbouring threads
            if ((seg & 1) == 0) reinterpret_cast<float*>(chunk + 2 * ACT_PLANE)[tok * 8 + (seg >> 1)] = sum;
        }
        if (seg == 0) {
            const int planes = p.bf3 ? 3 : 2;
            for (int pl = 0; pl < planes; ++pl)
                *reinterpret_cast<uint4*>(chunk + pl * ACT_PLANE + (tok * ACT_ROW_HALFS + 256) * 2) = make_uint4(0, 0, 0, 0);
        }
        if (over) atomicCAS(p.err, 0, DEV_ERR_OVERFLOW);
    }
}

dfl_status launch_glue(cudaStream_t st, const GlueParams& p, uint64_t k) {
    if (k == 0 || k % TILE_K) return fail(DFL_ERR_BAD_SHAPE, "glue: column count must be a positive multiple of 256");
    glue_kernel<<<(unsigned)(k / TILE_K), 256, 0, st>>>(p);
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

// ---- embedding rows ---------------------------------------------------------------
__global__ void embed_rows_kernel(int dtype, const uint8_t* __restrict__ ggml, uint64_t h, const int32_t* __restrict__ tokens,
                                  float* __restrict__ x, int ld) {
    const int tok = blockIdx.y;
    const uint64_t col = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (col >= h) return;
    const uint64_t row_bytes = h / 256 * (uint64_t)ggml_bytes_per_256(dtype);
    const uint8_t* seg = ggml + (uint64_t)tokens[tok] * row_bytes + (col >> 8) * (uint64_t)ggml_bytes_per_256(dtype);
    x[(uint64_t)tok * ld + col] = ggml_decode_elem(dtype, seg, (int)(col & 255));
}

dfl_status launch_embed_rows(cudaStream_t st, int dtype, const uint8_t* ggml, uint64_t h, const int32_t* tokens, int n_rows,
                             float* x, int ld) {
    if (h % 256 || ggml_bytes_per_256(dtype) == 0) return fail(DFL_ERR_UNSUPPORTED, "embed_rows: dtype or width");
    embed_rows_kernel<<<dim3((unsigned)((h + 255) / 256), (unsigned)n_rows), 256, 0, st>>>(dtype, ggml, h, tokens, x, ld);
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

// ---- small f32 matrices --------------------------------------------------------------
__global__ void __launch_bounds__(128) small_matmul_kernel(const float* __restrict__ w, const float* __restrict__ xn, int ld_xn,
                                                           int n_rows, uint64_t k, const float* __restrict__ sumsq, int n_sumsq,
                                                           float norm_k, float eps, float out_scale, float* __restrict__ out,
                                                           int ld_out) {
    const int j = blockIdx.x;
    float acc[MAX_ROWS];
#pragma unroll
    for (int r = 0; r < MAX_ROWS; ++r) acc[r] = 0.f;
    const float* wr = w + (uint64_t)j * k;
    for (uint64_t c = threadIdx.x; c < k; c += blockDim.x) {
        const float wv = wr[c];
#pragma unroll
        for (int r = 0; r < MAX_ROWS; ++r)
            if (r < n_rows) acc[r] = fmaf(wv, xn[(uint64_t)r * ld_xn + c], acc[r]);
    }
    __shared__ float red[4][MAX_ROWS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
    for (int r = 0; r < MAX_ROWS; ++r) {
        const float s = warp_sum(acc[r]);
        if (lane == 0) red[warp][r] = s;
    }
    __syncthreads();
    if (threadIdx.x < n_rows) {
        const int r = threadIdx.x;
        float s = red[0][r] + red[1][r] + red[2][r] + red[3][r];
        float sc = out_scale;
        if (sumsq) {
            float ss = 0.f;
            for (int i = 0; i < n_sumsq; ++i) ss += sumsq[i * MAX_ROWS + r];
            sc *= 1.0f / sqrtf(ss / norm_k + eps);
        }
        out[(uint64_t)r * ld_out + j] = s * sc;
    }
}

dfl_status launch_small_matmul(cudaStream_t st, const float* w, const float* xn, int ld_xn, int n_rows, uint64_t k, int n_out,
                               const GemmEpilogue& ep, float* out, int ld_out) {
    small_matmul_kernel<<<n_out, 128, 0, st>>>(w, xn, ld_xn, n_rows, k, ep.sumsq, ep.n_sumsq, ep.norm_k, ep.eps, ep.out_scale, out,
                                               ld_out);
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

}  // namespace dfl
