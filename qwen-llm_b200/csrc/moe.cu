// Routed-expert FFN, routing stage (reference: moe.metal:995-1089 kernels, metal_forward/moe.rs:349-751 host,
// CPU oracle forward.rs:749-824; the selection rule followed here is the CPU oracle's).
//
// One warp per token: softmax over all experts, the k experts with the largest probability
// (ties -> lower expert id) found with warp shuffles, weights re-normalised by their own sum
// (floored at 2^-14), written as one dense row route_w[token][expert] with zeros for the experts
// that were not chosen.  The expert GEMMs then run over all experts of the layer as two large
// few-row GEMMs (gate|up with n_out = E * F', down with n_in = E * F'), the SwiGLU glue multiplies
// each expert's inner columns by the token's route weight, so experts that were not chosen
// contribute exact zeros.  The shared expert's sigmoid gate comes from one extra router row.
#include "ops.cuh"

namespace dfl {

constexpr int MOE_MAX_EXPERTS = 1024;

__global__ void __launch_bounds__(32) moe_route_kernel(const float* logits, int ld, int n_expert, int n_used, int n_rows,
                                                       float* route_w, float* shared_gate,
                                                       int32_t* route_idx) {
    pdl_prologue();
    __shared__ float p[MOE_MAX_EXPERTS];
    const int tok = blockIdx.x, lane = threadIdx.x;
    float* wrow = route_w + (uint64_t)tok * n_expert;
    for (int i = lane; i < n_expert; i += 32) wrow[i] = 0.f;
    if (tok >= n_rows) {
        if (lane == 0) shared_gate[tok] = 0.f;
        for (int j = lane; j < n_used; j += 32) route_idx[tok * n_used + j] = -1;
        return;
    }
    const float* x = logits + (uint64_t)tok * ld;
    float mx = -INFINITY;
    for (int i = lane; i < n_expert; i += 32) mx = fmaxf(mx, x[i]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int i = lane; i < n_expert; i += 32) {
        const float e = expf(x[i] - mx);
        p[i] = e;
        sum += e;
    }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    for (int i = lane; i < n_expert; i += 32) p[i] *= inv;
    __syncwarp();
    float chosen_p = 0.f;   // lane j keeps the j-th choice
    int chosen_i = -1;
    for (int j = 0; j < n_used; ++j) {
        float best = -1.f;
        int bi = 0x7fffffff;
        for (int i = lane; i < n_expert; i += 32) {
            const float v = p[i];
            if (v > best || (v == best && i < bi)) { best = v; bi = i; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
        if (lane == (j & 31)) { chosen_p = best; chosen_i = bi; }
        if (lane == 0) p[bi] = -2.f;   // taken
        __syncwarp();
    }
    // sum of the chosen probabilities in choice order (the oracle's order)
    float wsum = 0.f;
    for (int j = 0; j < n_used && j < 32; ++j) wsum += __shfl_sync(0xffffffffu, chosen_p, j);
    wsum = fmaxf(wsum, 6.103515625e-05f);
    if (lane < n_used && chosen_i >= 0) {
        wrow[chosen_i] = chosen_p / wsum;
        route_idx[tok * n_used + lane] = chosen_i;
    }
    if (lane == 0) shared_gate[tok] = sigmoid_f(x[n_expert]);
}

dfl_status launch_moe_route(cudaStream_t st, const float* logits, int ld, int n_expert, int n_used, int n_rows, float* route_w,
                            float* shared_gate, int32_t* route_idx) {
    if (n_expert < 1 || n_expert > MOE_MAX_EXPERTS || n_used < 1 || n_used > 32 || n_used > n_expert)
        return fail(DFL_ERR_UNSUPPORTED, "moe_route: expert_count must be in [1, 1024] and expert_used_count in [1, 32]");
    launch_kf(16, moe_route_kernel, dim3(MAX_ROWS), dim3(32), 0, st, logits, ld, n_expert, n_used, n_rows, route_w, shared_gate, route_idx);
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

}  // namespace dfl
