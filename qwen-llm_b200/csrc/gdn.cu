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
#include <cooperative_groups.h>

#include "ops.cuh"

namespace dfl {

namespace cg = cooperative_groups;

// ---- front: conv1d(K=4) + SiLU over the block, q/k L2 norm -------------------------------
// grid = conv_dim / 128 (one q, k or v head per CTA), block 128: warp = group of four rows, lane = four channels
// (gdn_front_tile).  The conv state rows are read before the dependency wait: the previous pass wrote them and a
// pass begins with a host-to-device copy, so no kernel of this pass is their author.
__global__ void __launch_bounds__(128) gdn_front_kernel(const GdnFrontParams p) {
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31, head = blockIdx.x;
    float4 old[3] = {};
    if (w == 0) gdn_front_old_state(p, head, lane, old);
    pdl_prologue();
    __syncthreads();   // the old state has been read before any warp writes the new one
    gdn_front_tile(p, head, w, lane, old);
}

dfl_status launch_gdn_front_p(cudaStream_t st, const GdnFrontParams& p) {
    if (p.g.hd != 128 || p.g.conv_k != 4) return fail(DFL_ERR_UNSUPPORTED, "gdn: head_dim must be 128 and conv kernel 4");
    launch_k(gdn_front_kernel, dim3(p.g.conv_dim() / 128), dim3(128), 0, st, p);
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

dfl_status launch_gdn_front(cudaStream_t st, const GdnGeom& g, const float* part_qkv, int splits, int ld_part, int n_rows,
                            const float* conv_w, float* conv_state, float* qkv_raw, float* q_n, float* k_n, float* v, float* conv_pre) {
    GdnFrontParams p;
    p.g = g;
    p.part = part_qkv; p.splits = splits; p.ld_part = ld_part; p.n_rows = n_rows;
    p.conv_w = conv_w; p.conv_state = conv_state; p.qkv_raw = qkv_raw; p.q_n = q_n; p.k_n = k_n; p.v_out = v; p.conv_pre = conv_pre;
    return launch_gdn_front_p(st, p);
}

__global__ void gdn_conv_restore_kernel(int conv_dim, const float* conv_pre, const float* qkv_raw, int n_keep,
                                        float* conv_state) {
    pdl_prologue();
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
    launch_k(gdn_conv_restore_kernel, dim3((cd + 255) / 256), dim3(256), 0, st, cd, conv_pre, qkv_raw, n_keep, conv_state);
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

// One token of the recurrence for a warp's four state rows (lane owns columns lane + 32 j).
__device__ __forceinline__ void gdn_token_step(float (&S)[4][4], const float* k_row, const float* q_row, const float* v4, float gexp, float beta,
                                               int lane, float (&oo)[4]) {
    float kk[4], qq[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        kk[j] = k_row[lane + 32 * j];
        qq[j] = q_row[lane + 32 * j];
    }
    float sk[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        float p = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) p = fmaf(S[r][j], kk[j], p);
        sk[r] = p;
    }
#pragma unroll
    for (int of = 16; of > 0; of >>= 1)
#pragma unroll
        for (int r = 0; r < 4; ++r) sk[r] += __shfl_xor_sync(0xffffffffu, sk[r], of);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const float coeff = beta * (v4[r] - gexp * sk[r]);
        float p = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            S[r][j] = __fadd_rn(__fmul_rn(gexp, S[r][j]), __fmul_rn(coeff, kk[j]));
            p = fmaf(S[r][j], qq[j], p);
        }
        oo[r] = p;
    }
#pragma unroll
    for (int of = 16; of > 0; of >>= 1)
#pragma unroll
        for (int r = 0; r < 4; ++r) oo[r] += __shfl_xor_sync(0xffffffffu, oo[r], of);
}

// ---- scan (+ gated RMSNorm and activation packing) ------------------------------------------
// grid (n_v, 4) in clusters of four along y (the four quarters of a head's 128 value channels), block 256: warp
// owns 4 state rows (dv), lane owns columns dk = lane + 32 j.  The state rows are fetched before the dependency wait
// (the previous pass wrote them and a pass begins with a host-to-device copy, so no kernel of this pass is their
// author); the block's q, k, v rows, gate scalars and the z rows are staged in shared memory, so that the sequential
// part touches no global memory.  Per token (forward.rs:1054-1091): sk = S k (state before decay),
// coeff = beta (v - g sk), S = g S + coeff k, o = S q.
// With `acts` the kernel also finishes the layer's mixer: y = rmsnorm(o; eps * 128) * w * silu(z) over the head's 128
// channels (forward.rs:1093-1103), whose sum of squares the four CTAs of a cluster exchange through distributed shared
// memory and add in rank order, and packs its 32 columns of the out-projection's activations.  Without `acts` (the
// re-scan of a partial accept) only the state is advanced.
__global__ void __cluster_dims__(1, 4, 1) __launch_bounds__(256)
gdn_scan_kernel(GdnGeom g, const float* state_in, float* state_out, const float* q_n, const float* k_n, const float* v, const float* ab,
                const float* __restrict__ dt_bias, const float* __restrict__ a_log, int n_rows, const float* part_z, int z_splits, int ld_part,
                const float* __restrict__ norm_w, uint8_t* acts, int layout, int* err) {
    __shared__ float qs[MAX_ROWS][128], ks[MAX_ROWS][128], vs[MAX_ROWS][32], gs[MAX_ROWS], bs[MAX_ROWS], os[MAX_ROWS][32];
    __shared__ float zs[MAX_ROWS][32], ss_loc[MAX_ROWS], scale_s[MAX_ROWS];
    const int h = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hk = h % g.n_k;
    const int dv_cta = blockIdx.y * 32, dv0 = dv_cta + warp * 4;
    float S[4][4];
    const float* sin = state_in + ((uint64_t)h * 128 + dv0) * 128;
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int j = 0; j < 4; ++j) S[r][j] = __ldcg(sin + r * 128 + lane + 32 * j);
    const float dtb = dt_bias[h], alog = a_log[h];
    pdl_prologue();
    for (int idx = threadIdx.x; idx < n_rows * 128; idx += 256) {
        const int i = idx >> 7, d = idx & 127;
        qs[i][d] = q_n[((uint64_t)i * g.n_k + hk) * 128 + d];
        ks[i][d] = k_n[((uint64_t)i * g.n_k + hk) * 128 + d];
    }
    for (int idx = threadIdx.x; idx < n_rows * 32; idx += 256) {
        const int i = idx >> 5, d = idx & 31;
        vs[i][d] = v[((uint64_t)i * g.n_v + h) * 128 + dv_cta + d];
    }
    if (threadIdx.x < n_rows) {
        // gate inputs: ab[i][0..n_v) = alpha projection, ab[i][n_v..2 n_v) = beta projection
        const int i = threadIdx.x;
        const float alpha = ab[(uint64_t)i * (2 * g.n_v) + h] + dtb;
        gs[i] = expf(softplus_f(alpha) * alog);
        bs[i] = sigmoid_f(ab[(uint64_t)i * (2 * g.n_v) + g.n_v + h]);
    }
    if (acts) {
        // z = the z projection's split-K partials summed in slice order; two tokens' worth per pass of the CTA
        for (int idx = threadIdx.x; idx < n_rows * 32; idx += 256) {
            const int i = idx >> 5, d = idx & 31;
            const float* zp = part_z + (uint64_t)i * ld_part + h * 128 + dv_cta + d;
            float z = 0.f;
#pragma unroll 4
            for (int s = 0; s < z_splits; ++s) z += zp[(uint64_t)s * MAX_ROWS * ld_part];
            zs[i][d] = z;
        }
    }
    __syncthreads();
    for (int i = 0; i < n_rows; ++i) {
        float oo[4];
        gdn_token_step(S, ks[i], qs[i], &vs[i][warp * 4], gs[i], bs[i], lane, oo);
        if (lane < 4) os[i][warp * 4 + lane] = lane == 0 ? oo[0] : lane == 1 ? oo[1] : lane == 2 ? oo[2] : oo[3];
    }
    float* sout = state_out + ((uint64_t)h * 128 + dv0) * 128;
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int j = 0; j < 4; ++j) sout[r * 128 + lane + 32 * j] = S[r][j];
    if (!acts) return;   // uniform over the grid: no CTA of any cluster reaches the cluster barriers below
    __syncthreads();
    // this quarter's share of each token's sum of squares (two tokens per warp)
    for (int i = warp; i < MAX_ROWS; i += 8) {
        const float x = i < n_rows ? os[i][lane] : 0.f;
        const float sq = warp_sum(x * x);
        if (lane == 0) ss_loc[i] = sq;
    }
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();   // every quarter's shares are written
    if (threadIdx.x < MAX_ROWS) {
        float tot = 0.f;
#pragma unroll
        for (unsigned r = 0; r < 4; ++r) tot += *cluster.map_shared_rank(&ss_loc[threadIdx.x], r);   // rank order: the same sum in all four CTAs
        scale_s[threadIdx.x] = 1.0f / sqrtf(tot / 128.f + 1e-6f * 128.f);   // eps = RMS_EPS * head_dim (forward.rs:1098)
    }
    cluster.sync();   // scale_s visible in the CTA; nobody leaves while its shares may still be read
    if (threadIdx.x < 128) {
        const int tok = threadIdx.x >> 3, quad = threadIdx.x & 7;
        const int col0 = h * 128 + dv_cta + quad * 4;
        float y[4] = {0.f, 0.f, 0.f, 0.f};
        if (tok < n_rows) {
            const float4 nw = *reinterpret_cast<const float4*>(norm_w + dv_cta + quad * 4);
            const float sc = scale_s[tok];
            y[0] = os[tok][quad * 4 + 0] * sc * nw.x * silu_f(zs[tok][quad * 4 + 0]);
            y[1] = os[tok][quad * 4 + 1] * sc * nw.y * silu_f(zs[tok][quad * 4 + 1]);
            y[2] = os[tok][quad * 4 + 2] * sc * nw.z * silu_f(zs[tok][quad * 4 + 2]);
            y[3] = os[tok][quad * 4 + 3] * sc * nw.w * silu_f(zs[tok][quad * 4 + 3]);
        }
        uint8_t* chunk = acts + (uint64_t)(col0 >> 8) * act_chunk_dev(layout);
        bool over = false;
        pack_quad_any(chunk, layout, tok, col0 & 255, y, over);
        if (layout == ACT_F16 || layout == ACT_TS) {
            float sum = y[0] + y[1] + y[2] + y[3];   // the CTA's 32 channels are one 32-column sub-block: eight neighbouring threads
#pragma unroll
            for (int of = 4; of > 0; of >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, of);
            if (quad == 0) store_subsum(chunk, layout, tok, (col0 & 255) >> 5, sum, over);
        }
        if (over) atomicCAS(err, 0, DEV_ERR_OVERFLOW);
    }
}

dfl_status launch_gdn_scan(cudaStream_t st, const GdnGeom& g, const float* state_in, float* state_out, const float* q_n,
                           const float* k_n, const float* v, const float* ab, const float* dt_bias, const float* a_log, int n_rows,
                           const float* part_z, int z_splits, int ld_part, const float* norm_w, uint8_t* acts, int act_layout, int* err) {
    launch_k(gdn_scan_kernel, dim3(dim3((unsigned)g.n_v, 4)), dim3(256), 0, st, g, state_in, state_out, q_n, k_n, v, ab, dt_bias, a_log, n_rows,
              part_z, z_splits, ld_part, norm_w, acts, act_layout, err);
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

}  // namespace dfl
