// Gated-delta-net block of the verify pass (oracle: Forward::gdn_step,
// crates/qwen-llm/src/forward.rs:940-1107; reference GPU path metal_dflash.rs:9421-9777,
// kernels/ssm_conv.metal:225-277,305-346, kernels/gated_delta_net.metal:382-470).
//
// Rollback design: the recurrence reads the state from one buffer and writes the advanced
// state to another, and the block's raw qkv rows and gate inputs stay in the scratch.  A full
// accept just swaps the two buffers; a partial accept re-runs the same scan device code for
// the first n_keep tokens from the untouched pre-block state, which reproduces the sequential
// state bit for bit without the reference's per-token state checkpoints
// (metal_dflash.rs:5863-5896: n_gdn x N x state bytes written every verify).
#include "ops.cuh"

namespace dfl {

// ---- front: conv1d(K=4) + SiLU over the block, q/k L2 norm -------------------------------
// grid = conv_dim / 128 (one q, k or v head per CTA), block 128 (one channel per thread).
__global__ void __launch_bounds__(128) gdn_front_kernel(GdnGeom g, const float* __restrict__ part, int splits, int ld_part, int n_rows,
                                                        const float* __restrict__ conv_w, float* __restrict__ conv_state,
                                                        float* __restrict__ qkv_raw, float* __restrict__ q_n, float* __restrict__ k_n,
                                                        float* __restrict__ v_out) {
    const int conv_dim = g.conv_dim();
    const int c = blockIdx.x * 128 + threadIdx.x;
    const int head = blockIdx.x;  // heads of 128 channels: [0, n_k) q, [n_k, 2 n_k) k, rest v
    float w0 = conv_w[c * 4 + 0], w1 = conv_w[c * 4 + 1], w2 = conv_w[c * 4 + 2], w3 = conv_w[c * 4 + 3];
    float h0 = conv_state[0 * conv_dim + c], h1 = conv_state[1 * conv_dim + c], h2 = conv_state[2 * conv_dim + c];
    __shared__ float red[4];
    const bool is_v = head >= 2 * g.n_k;
    float* dst = is_v ? v_out + (uint64_t)(head - 2 * g.n_k) * 128 + threadIdx.x
                      : (head < g.n_k ? q_n + (uint64_t)head * 128 + threadIdx.x : k_n + (uint64_t)(head - g.n_k) * 128 + threadIdx.x);
    const int dst_ld = is_v ? g.n_v * 128 : g.n_k * 128;
    for (int i = 0; i < n_rows; ++i) {
        float x = 0.f;
        for (int s = 0; s < splits; ++s) x += part[((uint64_t)s * MAX_ROWS + i) * ld_part + c];
        qkv_raw[(uint64_t)i * conv_dim + c] = x;
        // s = sum_k w[k] * window[k], k ascending (forward.rs:1000-1010)
        float sacc = 0.f;
        sacc += w0 * h0;
        sacc += w1 * h1;
        sacc += w2 * h2;
        sacc += w3 * x;
        float y = silu_f(sacc);
        h0 = h1; h1 = h2; h2 = x;
        if (!is_v) {
            // y / max(||y||, eps) over the head's 128 channels (forward.rs:1269-1275)
            float sq = warp_sum(y * y);
            __syncthreads();
            if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sq;
            __syncthreads();
            const float tot = red[0] + red[1] + red[2] + red[3];
            y *= 1.0f / fmaxf(sqrtf(tot), 1e-6f);
        }
        dst[(uint64_t)i * dst_ld] = y;
    }
    conv_state[0 * conv_dim + c] = h0;
    conv_state[1 * conv_dim + c] = h1;
    conv_state[2 * conv_dim + c] = h2;
}

dfl_status launch_gdn_front(cudaStream_t st, const GdnGeom& g, const float* part_qkv, int splits, int ld_part, int n_rows,
                            const float* conv_w, float* conv_state, float* qkv_raw, float* q_n, float* k_n, float* v) {
    if (g.hd != 128 || g.conv_k != 4) return fail(DFL_ERR_UNSUPPORTED, "gdn: head_dim must be 128 and conv kernel 4");
    gdn_front_kernel<<<g.conv_dim() / 128, 128, 0, st>>>(g, part_qkv, splits, ld_part, n_rows, conv_w, conv_state, qkv_raw, q_n, k_n, v);
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

__global__ void gdn_conv_restore_kernel(int conv_dim, const float* __restrict__ conv_pre, const float* __restrict__ qkv_raw, int n_keep,
                                        float* __restrict__ conv_state) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= conv_dim) return;
    // rows of the virtual sequence {pre[0], pre[1], pre[2], raw[0], ..., raw[n_keep-1]}; keep the last three
#pragma unroll
    for (int t = 0; t < 3; ++t) {
        const int idx = n_keep + t;  // index into the virtual sequence
        conv_state[t * conv_dim + c] = idx < 3 ? conv_pre[idx * conv_dim + c] : qkv_raw[(uint64_t)(idx - 3) * conv_dim + c];
    }
}
dfl_status launch_gdn_conv_restore(cudaStream_t st, const GdnGeom& g, const float* conv_pre, const float* qkv_raw, int n_keep,
                                   float* conv_state) {
    const int cd = g.conv_dim();
    gdn_conv_restore_kernel<<<(cd + 255) / 256, 256, 0, st>>>(cd, conv_pre, qkv_raw, n_keep, conv_state);
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

// ---- scan --------------------------------------------------------------------------------
// grid (n_v, 4), block 256: warp owns 4 state rows (dv), lane owns columns dk = lane + 32 j.
// Per token (forward.rs:1054-1091): sk = S k (state before decay), coeff = beta (v - g sk),
// S = g S + coeff k, o = S q.
__global__ void __launch_bounds__(256) gdn_scan_kernel(GdnGeom g, const float* __restrict__ state_in, float* __restrict__ state_out,
                                                       const float* __restrict__ q_n, const float* __restrict__ k_n,
                                                       const float* __restrict__ v, const float* __restrict__ ab,
                                                       const float* __restrict__ dt_bias, const float* __restrict__ a_log, int n_rows,
                                                       float* __restrict__ o) {
    const int h = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hk = h % g.n_k;
    const int dv0 = blockIdx.y * 32 + warp * 4;
    float S[4][4];
    const float* sin = state_in + ((uint64_t)h * 128 + dv0) * 128;
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int j = 0; j < 4; ++j) S[r][j] = sin[r * 128 + lane + 32 * j];
    const float dtb = dt_bias[h], al = a_log[h];
    for (int i = 0; i < n_rows; ++i) {
        // gate inputs: ab[i][0..n_v) = alpha projection, ab[i][n_v..2 n_v) = beta projection
        const float alpha = ab[(uint64_t)i * (2 * g.n_v) + h] + dtb;
        const float gexp = expf(softplus_f(alpha) * al);
        const float beta = sigmoid_f(ab[(uint64_t)i * (2 * g.n_v) + g.n_v + h]);
        float kk[4], qq[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            kk[j] = k_n[((uint64_t)i * g.n_k + hk) * 128 + lane + 32 * j];
            qq[j] = q_n[((uint64_t)i * g.n_k + hk) * 128 + lane + 32 * j];
        }
        float sk[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            float p = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) p = fmaf(S[r][j], kk[j], p);
            sk[r] = warp_sum(p);
        }
        float oo[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const float vv = v[((uint64_t)i * g.n_v + h) * 128 + dv0 + r];
            const float coeff = beta * (vv - gexp * sk[r]);
            float p = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                S[r][j] = __fadd_rn(__fmul_rn(gexp, S[r][j]), __fmul_rn(coeff, kk[j]));
                p = fmaf(S[r][j], qq[j], p);
            }
            oo[r] = warp_sum(p);
        }
        if (o && lane < 4) o[((uint64_t)i * g.n_v + h) * 128 + dv0 + lane] = lane == 0 ? oo[0] : lane == 1 ? oo[1] : lane == 2 ? oo[2] : oo[3];
    }
    float* sout = state_out + ((uint64_t)h * 128 + dv0) * 128;
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int j = 0; j < 4; ++j) sout[r * 128 + lane + 32 * j] = S[r][j];
}

dfl_status launch_gdn_scan(cudaStream_t st, const GdnGeom& g, const float* state_in, float* state_out, const float* q_n,
                           const float* k_n, const float* v, const float* ab, const float* dt_bias, const float* a_log, int n_rows,
                           float* o) {
    gdn_scan_kernel<<<dim3((unsigned)g.n_v, 4), 256, 0, st>>>(g, state_in, state_out, q_n, k_n, v, ab, dt_bias, a_log, n_rows, o);
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

// ---- post: gated RMSNorm + activation packing ----------------------------------------------
// grid (n_v, 16), block 32: one warp per (head, token); lane owns 4 consecutive channels.
__global__ void __launch_bounds__(32) gdn_post_kernel(GdnGeom g, const float* __restrict__ o, const float* __restrict__ part_z, int splits,
                                                      int ld_part, const float* __restrict__ norm_w, int n_rows, uint8_t* acts, int bf3,
                                                      int* err) {
    const int h = blockIdx.x, tok = blockIdx.y, lane = threadIdx.x;
    const int col0 = h * 128 + lane * 4;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (tok < n_rows) {
        const float4 ov = *reinterpret_cast<const float4*>(o + (uint64_t)tok * (g.n_v * 128) + col0);
        float z[4] = {0.f, 0.f, 0.f, 0.f};
        for (int s = 0; s < splits; ++s) {
            const float4 zz = *reinterpret_cast<const float4*>(part_z + ((uint64_t)s * MAX_ROWS + tok) * ld_part + col0);
            z[0] += zz.x; z[1] += zz.y; z[2] += zz.z; z[3] += zz.w;
        }
        const float ss = warp_sum(ov.x * ov.x + ov.y * ov.y + ov.z * ov.z + ov.w * ov.w);
        const float scale = 1.0f / sqrtf(ss / 128.f + 1e-6f * 128.f);  // eps = RMS_EPS * head_dim (forward.rs:1098)
        const float4 nw = *reinterpret_cast<const float4*>(norm_w + lane * 4);
        v[0] = ov.x * scale * nw.x * silu_f(z[0]);
        v[1] = ov.y * scale * nw.y * silu_f(z[1]);
        v[2] = ov.z * scale * nw.z * silu_f(z[2]);
        v[3] = ov.w * scale * nw.w * silu_f(z[3]);
    }
    uint8_t* chunk = acts + (uint64_t)(col0 >> 8) * (bf3 ? ACTB3_CHUNK : ACT16_CHUNK);
    bool over = false;
    pack_quad(chunk, bf3 != 0, tok, col0 & 255, v, over);
    if (!bf3) {
        float sum = v[0] + v[1] + v[2] + v[3];
#pragma unroll
        for (int of = 4; of > 0; of >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, of);
        if ((lane & 7) == 0) reinterpret_cast<float*>(chunk + 2 * ACT_PLANE)[tok * 8 + ((col0 & 255) >> 5)] = sum;
    }
    if (over) atomicCAS(err, 0, DEV_ERR_OVERFLOW);
}

dfl_status launch_gdn_post(cudaStream_t st, const GdnGeom& g, const float* o, const float* part_z, int splits, int ld_part,
                           const float* norm_w, int n_rows, uint8_t* acts, bool bf3, int* err) {
    gdn_post_kernel<<<dim3((unsigned)g.n_v, MAX_ROWS), 32, 0, st>>>(g, o, part_z, splits, ld_part, norm_w, n_rows, acts, bf3 ? 1 : 0, err);
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

}  // namespace dfl
