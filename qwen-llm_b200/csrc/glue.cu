// Element-wise kernels between two GEMMs: split-K reduction, residual add, SwiGLU, folding of
// the RMSNorm weight, hidden-state capture and packing of the next GEMM's activations, in one
// pass.  Replaces the reference's separate kernel_add_inplace_f32 / kernel_silu_mul_f32 /
// kernel_rms_norm_batched_f32 launches (kernels/elementwise.metal:89,193; rms_norm.metal:48).
//
// RMSNorm is split so that no row-wide reduction sits on the critical path: this kernel
// multiplies by the norm weight and emits per-64-column partial sums of squares; the
// consuming GEMM multiplies its result by 1/sqrt(mean(x^2) + eps) per token.
#include "ops.cuh"

namespace dfl {

// grid = k / 64, block 256: thread = (token = tid / 16, four consecutive columns).  One float4 per
// split per thread keeps every global load of the kernel independent (one latency round).
__global__ void __launch_bounds__(256) glue_kernel(const GlueParams p) {
    pdl_prologue();
    const int n_splits = p.splits_dev ? p.splits + *p.splits_dev : p.splits;
    const int cb = blockIdx.x, tok = threadIdx.x >> 4, quad = threadIdx.x & 15;
    const int col0 = cb * GLUE_COLS + quad * 4;
    const bool live = tok < p.n_rows;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (live) {
        if (p.mode == GLUE_SWIGLU) {
            // route weight of this row for the expert the columns belong to (1 without routing); a row that did not
            // choose the expert gets exact zeros and its partial sums - possibly stale - are not even read
            float w = 1.f;
            if (p.route_w) w = col0 < p.route_n * p.route_f ? p.route_w[tok * p.route_e + p.route_e0 + col0 / p.route_f] : p.route_sg[tok];
            if (w != 0.f) {
                float g[4] = {0.f, 0.f, 0.f, 0.f}, u[4] = {0.f, 0.f, 0.f, 0.f};
                const float* base = p.part + (uint64_t)tok * p.ld_part + col0;
                const uint64_t stride = (uint64_t)MAX_ROWS * p.ld_part;
#pragma unroll 4
                for (int s = 0; s < n_splits; ++s) {
                    const float4 a = *reinterpret_cast<const float4*>(base + s * stride);
                    const float4 b = *reinterpret_cast<const float4*>(base + s * stride + p.swiglu_f);
                    g[0] += a.x; g[1] += a.y; g[2] += a.z; g[3] += a.w;
                    u[0] += b.x; u[1] += b.y; u[2] += b.z; u[3] += b.w;
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) v[j] = silu_f(g[j]) * u[j];
                if (p.route_w) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) v[j] *= w;
                }
            }
        } else {
            float4 xv = make_float4(0.f, 0.f, 0.f, 0.f);
            if (p.x) xv = *reinterpret_cast<const float4*>(p.x + (uint64_t)tok * p.ld_x + col0);
            if (p.mode == GLUE_RESID && p.part) {
                // sum the split-K partials first (fixed order), then add to the residual
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
                const float* base = p.part + (uint64_t)tok * p.ld_part + col0;
                const uint64_t stride = (uint64_t)MAX_ROWS * p.ld_part;
#pragma unroll 4
                for (int s = 0; s < n_splits; ++s) {
                    const float4 a = *reinterpret_cast<const float4*>(base + s * stride);
                    acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
                }
                v[0] = xv.x + acc[0]; v[1] = xv.y + acc[1]; v[2] = xv.z + acc[2]; v[3] = xv.w + acc[3];
                if (p.x) *reinterpret_cast<float4*>(p.x + (uint64_t)tok * p.ld_x + col0) = make_float4(v[0], v[1], v[2], v[3]);
            } else {
                v[0] = xv.x; v[1] = xv.y; v[2] = xv.z; v[3] = xv.w;
            }
        }
        if (p.capture)
            *reinterpret_cast<float4*>(p.capture + (uint64_t)tok * p.ld_capture + col0) = make_float4(v[0], v[1], v[2], v[3]);
    }
    if (p.sumsq) {
        float ss = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (quad == 0) p.sumsq[cb * MAX_ROWS + tok] = ss;
    }
    if (p.mul_w) {
        const float4 w = *reinterpret_cast<const float4*>(p.mul_w + col0);
        v[0] *= w.x; v[1] *= w.y; v[2] *= w.z; v[3] *= w.w;
    }
    if (p.pre_scale != 1.f) {
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] *= p.pre_scale;
    }
    if (p.xn && live) *reinterpret_cast<float4*>(p.xn + (uint64_t)tok * p.ld_xn + col0) = make_float4(v[0], v[1], v[2], v[3]);
    if (p.acts) {
        uint8_t* chunk = p.acts + (uint64_t)(col0 >> 8) * act_chunk_dev(p.bf3);
        bool over = false;
        pack_quad_any(chunk, p.bf3, tok, col0 & 255, v, over);
        if ((p.bf3 == ACT_F16 || p.bf3 == ACT_TS)) {
            float sum = v[0] + v[1] + v[2] + v[3];  // 32-column sub-block = eight neighbouring threads
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            if ((quad & 7) == 0) store_subsum(chunk, p.bf3, tok, (col0 & 255) >> 5, sum, over);
        }
        if (over) atomicCAS(p.err, 0, DEV_ERR_OVERFLOW);
    }
}

dfl_status launch_glue(cudaStream_t st, const GlueParams& p, uint64_t k) {
    if (k == 0 || k % TILE_K) return fail(DFL_ERR_BAD_SHAPE, "glue: column count must be a positive multiple of 256");
    launch_kf(2, glue_kernel, dim3((unsigned)(k / GLUE_COLS)), dim3(256), 0, st, p);
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

// ---- embedding rows ---------------------------------------------------------------
__global__ void embed_rows_kernel(int dtype, const uint8_t* __restrict__ ggml, uint64_t h, const int32_t* tokens,
                                  float* x, int ld) {
    pdl_prologue();
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
    launch_kf(2, embed_rows_kernel, dim3(dim3((unsigned)((h + 255) / 256), (unsigned)n_rows)), dim3(256), 0, st, dtype, ggml, h, tokens, x, ld);
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

// ---- small f32 matrices --------------------------------------------------------------
// One CTA of 512 threads per output column; each thread takes float4 slices of the row so that all
// of its loads are independent, then a fixed-order block reduction per token.
__global__ void __launch_bounds__(512) small_matmul_kernel(const float* __restrict__ w, const float* xn, int ld_xn,
                                                           int n_rows, uint64_t k, const float* sumsq, int n_sumsq,
                                                           float norm_k, float eps, float out_scale, float* out,
                                                           int ld_out) {
    pdl_prologue();
    const int j = blockIdx.x;
    // per-token output scale first (16 threads per token, fixed tree), so that it overlaps the weight loads
    __shared__ float scale_s[MAX_ROWS];
    if (threadIdx.x < 256) {
        const int tok = threadIdx.x >> 4, part = threadIdx.x & 15;
        float ss = 0.f;
        if (sumsq)
            for (int i = part; i < n_sumsq; i += 16) ss += sumsq[i * MAX_ROWS + tok];
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (part == 0) scale_s[tok] = sumsq ? out_scale * (1.0f / sqrtf(ss / norm_k + eps)) : out_scale;
    }
    float acc[MAX_ROWS];
#pragma unroll
    for (int r = 0; r < MAX_ROWS; ++r) acc[r] = 0.f;
    const float* wr = w + (uint64_t)j * k;
    for (uint64_t c = (uint64_t)threadIdx.x * 4; c < k; c += 512 * 4) {
        const float4 wv = *reinterpret_cast<const float4*>(wr + c);
#pragma unroll
        for (int r = 0; r < MAX_ROWS; ++r) {
            if (r < n_rows) {
                const float4 xv = *reinterpret_cast<const float4*>(xn + (uint64_t)r * ld_xn + c);
                acc[r] = fmaf(wv.w, xv.w, fmaf(wv.z, xv.z, fmaf(wv.y, xv.y, fmaf(wv.x, xv.x, acc[r]))));
            }
        }
    }
    __shared__ float red[16][MAX_ROWS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
    for (int r = 0; r < MAX_ROWS; ++r) {
        const float s = warp_sum(acc[r]);
        if (lane == 0) red[warp][r] = s;
    }
    __syncthreads();
    if (threadIdx.x < n_rows) {
        const int r = threadIdx.x;
        float s = 0.f;
#pragma unroll
        for (int wv = 0; wv < 16; ++wv) s += red[wv][r];
        out[(uint64_t)r * ld_out + j] = s * scale_s[r];
    }
}

dfl_status launch_small_matmul(cudaStream_t st, const float* w, const float* xn, int ld_xn, int n_rows, uint64_t k, int n_out,
                               const GemmEpilogue& ep, float* out, int ld_out) {
    if (k % 4) return fail(DFL_ERR_BAD_SHAPE, "small_matmul: k must be a multiple of 4");
    launch_kf(2, small_matmul_kernel, dim3(n_out), dim3(512), 0, st, w, xn, ld_xn, n_rows, k, ep.sumsq, ep.n_sumsq, ep.norm_k, ep.eps, ep.out_scale, out,
                                               ld_out);
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

}  // namespace dfl
