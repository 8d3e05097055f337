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
    glue_quad(p, n_splits, blockIdx.x, threadIdx.x >> 4, threadIdx.x & 15);
}

dfl_status launch_glue(cudaStream_t st, const GlueParams& p, uint64_t k) {
    if (k == 0 || k % TILE_K) return fail(DFL_ERR_BAD_SHAPE, "glue: column count must be a positive multiple of 256");
    launch_k(glue_kernel, dim3((unsigned)(k / GLUE_COLS)), dim3(256), 0, st, p);
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
    launch_k(embed_rows_kernel, dim3(dim3((unsigned)((h + 255) / 256), (unsigned)n_rows)), dim3(256), 0, st, dtype, ggml, h, tokens, x, ld);
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
    launch_k(small_matmul_kernel, dim3(n_out), dim3(512), 0, st, w, xn, ld_xn, n_rows, k, ep.sumsq, ep.n_sumsq, ep.norm_k, ep.eps, ep.out_scale, out,
                                               ld_out);
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

}  // namespace dfl
