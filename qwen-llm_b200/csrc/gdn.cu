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

// One token of the recurrence for one state row shared by eight lanes: lane group member lg owns the sixteen columns
// dk = 32 j + 4 lg + c (j, c < 4), so that the eight lanes of a row read 128 contiguous bytes of k and q per step.
// The two row sums go through three shuffle levels each.
__device__ __forceinline__ float gdn_token_step(float (&S)[16], const float* k_row, const float* q_row, float v, float gexp, float beta, int lg) {
    float kk[16], qq[16];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float4 k4 = *reinterpret_cast<const float4*>(k_row + 32 * j + 4 * lg);
        const float4 q4 = *reinterpret_cast<const float4*>(q_row + 32 * j + 4 * lg);
        kk[4 * j] = k4.x; kk[4 * j + 1] = k4.y; kk[4 * j + 2] = k4.z; kk[4 * j + 3] = k4.w;
        qq[4 * j] = q4.x; qq[4 * j + 1] = q4.y; qq[4 * j + 2] = q4.z; qq[4 * j + 3] = q4.w;
    }
    float p[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        p[j] = S[4 * j] * kk[4 * j];
#pragma unroll
        for (int c = 1; c < 4; ++c) p[j] = fmaf(S[4 * j + c], kk[4 * j + c], p[j]);
    }
    float sk = (p[0] + p[1]) + (p[2] + p[3]);
#pragma unroll
    for (int of = 4; of > 0; of >>= 1) sk += __shfl_xor_sync(0xffffffffu, sk, of);
    const float coeff = beta * (v - gexp * sk);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int e = 4 * j + c;
            S[e] = __fadd_rn(__fmul_rn(gexp, S[e]), __fmul_rn(coeff, kk[e]));
        }
        p[j] = S[4 * j] * qq[4 * j];
#pragma unroll
        for (int c = 1; c < 4; ++c) p[j] = fmaf(S[4 * j + c], qq[4 * j + c], p[j]);
    }
    float o = (p[0] + p[1]) + (p[2] + p[3]);
#pragma unroll
    for (int of = 4; of > 0; of >>= 1) o += __shfl_xor_sync(0xffffffffu, o, of);
    return o;
}

// ---- scan (+ gated RMSNorm and activation packing) ------------------------------------------
// grid (n_v, 4) in clusters of four along y (the four quarters of a head's 128 value channels), block 256: a warp
// owns 4 state rows (dv), eight lanes per row, sixteen columns (dk) per lane.  The state rows are fetched before the
// dependency wait (the previous pass wrote them and a pass begins with a host-to-device copy, so no kernel of this
// pass is their author); the block's q, k, v rows and gate scalars are staged in shared memory, so that the
// sequential part touches no global memory; the z rows are requested before the token loop and used after it.
// Per token (forward.rs:1054-1091): sk = S k (state before decay), coeff = beta (v - g sk), S = g S + coeff k, o = S q.
// With `acts` the kernel also finishes the layer's mixer: y = rmsnorm(o; eps * 128) * w * silu(z) over the head's 128
// channels (forward.rs:1093-1103).  Each CTA writes its quarter's share of every token's sum of squares into all four
// CTAs of its cluster through distributed shared memory, one cluster barrier later each adds the four shares in rank
// order, and packs its 32 columns of the out-projection's activations.  Without `acts` (the re-scan of a partial
// accept) only the state is advanced.
__global__ void __cluster_dims__(1, 4, 1) __launch_bounds__(256)
gdn_scan_kernel(GdnGeom g, const float* state_in, float* state_out, const float* q_n, const float* k_n, const float* v, const float* ab,
                const float* __restrict__ dt_bias, const float* __restrict__ a_log, int n_rows, const float* part_z, int z_splits, int ld_part,
                const float* __restrict__ norm_w, uint8_t* acts, int layout, int* err) {
    __shared__ __align__(16) float qs[MAX_ROWS][128], ks[MAX_ROWS][128];
    __shared__ float vs[MAX_ROWS][32], gs[MAX_ROWS], bs[MAX_ROWS], os[MAX_ROWS][32];
    __shared__ float ss_all[4][MAX_ROWS];   // [cluster rank][token]: every quarter's share of the sum of squares
    cg::cluster_group cluster = cg::this_cluster();
    if (acts) cluster.barrier_arrive();   // matched by the wait before the first write into another CTA's shared memory
    const int h = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rr = lane >> 3, lg = lane & 7;
    const int hk = h % g.n_k;
    const int dv_cta = blockIdx.y * 32, dv = dv_cta + warp * 4 + rr;
    float S[16];
    const float* sin = state_in + ((uint64_t)h * 128 + dv) * 128 + 4 * lg;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float4 s4 = __ldcg(reinterpret_cast<const float4*>(sin + 32 * j));
        S[4 * j] = s4.x; S[4 * j + 1] = s4.y; S[4 * j + 2] = s4.z; S[4 * j + 3] = s4.w;
    }
    const float dtb = dt_bias[h], alog = a_log[h];
    pdl_prologue();
    for (int idx = threadIdx.x; idx < n_rows * 32; idx += 256) {
        const int i = idx >> 5, d4 = (idx & 31) * 4;
        *reinterpret_cast<float4*>(&qs[i][d4]) = *reinterpret_cast<const float4*>(q_n + ((uint64_t)i * g.n_k + hk) * 128 + d4);
        *reinterpret_cast<float4*>(&ks[i][d4]) = *reinterpret_cast<const float4*>(k_n + ((uint64_t)i * g.n_k + hk) * 128 + d4);
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
    // the finishing threads (token, four channels) fetch their z values now: the z projection's split-K partials
    // summed in slice order; the loads complete under the token loop
    const int ftok = threadIdx.x >> 3, fquad = threadIdx.x & 7;
    float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (acts && threadIdx.x < 128 && ftok < n_rows) {
        const float* zp = part_z + (uint64_t)ftok * ld_part + h * 128 + dv_cta + fquad * 4;
#pragma unroll 4
        for (int s = 0; s < z_splits; ++s) {
            const float4 t = __ldcg(reinterpret_cast<const float4*>(zp + (uint64_t)s * MAX_ROWS * ld_part));
            z4.x += t.x; z4.y += t.y; z4.z += t.z; z4.w += t.w;
        }
    }
    __syncthreads();
#pragma unroll 2
    for (int i = 0; i < n_rows; ++i) {
        const float o = gdn_token_step(S, ks[i], qs[i], vs[i][warp * 4 + rr], gs[i], bs[i], lg);
        if (lg == 0) os[i][warp * 4 + rr] = o;
    }
    float* sout = state_out + ((uint64_t)h * 128 + dv) * 128 + 4 * lg;
#pragma unroll
    for (int j = 0; j < 4; ++j) *reinterpret_cast<float4*>(sout + 32 * j) = make_float4(S[4 * j], S[4 * j + 1], S[4 * j + 2], S[4 * j + 3]);
    if (!acts) return;   // uniform over the grid: no CTA of any cluster reaches the cluster barriers below
    __syncthreads();
    cluster.barrier_wait();   // every CTA of the cluster has started: its shared memory may be written
    // this quarter's share of each token's sum of squares (two tokens per warp), written into all four CTAs
    const unsigned my_rank = cluster.block_rank();
    for (int i = warp; i < MAX_ROWS; i += 8) {
        const float x = i < n_rows ? os[i][lane] : 0.f;
        const float sq = warp_sum(x * x);
        if (lane < 4) *cluster.map_shared_rank(&ss_all[my_rank][i], (unsigned)lane) = sq;
    }
    cluster.sync();   // all shares have arrived; nothing is written into another CTA after this point
    if (threadIdx.x < 128) {
        const int tok = ftok, quad = fquad;
        const int col0 = h * 128 + dv_cta + quad * 4;
        float y[4] = {0.f, 0.f, 0.f, 0.f};
        if (tok < n_rows) {
            const float tot = ((ss_all[0][tok] + ss_all[1][tok]) + ss_all[2][tok]) + ss_all[3][tok];   // rank order: the same sum in all four CTAs
            const float sc = 1.0f / sqrtf(tot / 128.f + 1e-6f * 128.f);   // eps = RMS_EPS * head_dim (forward.rs:1098)
            const float4 nw = *reinterpret_cast<const float4*>(norm_w + dv_cta + quad * 4);
            y[0] = os[tok][quad * 4 + 0] * sc * nw.x * silu_f(z4.x);
            y[1] = os[tok][quad * 4 + 1] * sc * nw.y * silu_f(z4.y);
            y[2] = os[tok][quad * 4 + 2] * sc * nw.z * silu_f(z4.z);
            y[3] = os[tok][quad * 4 + 3] * sc * nw.w * silu_f(z4.w);
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
