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

// routing of one row by one warp; p = n_expert floats of shared memory of its own
__device__ __forceinline__ void moe_route_row(float* p, int tok, int lane, const float* logits, int ld, int n_expert, int n_used, int n_rows,
                                              float* route_w, float* shared_gate, int32_t* route_idx, int* err) {
    float* wrow = route_w + (uint64_t)tok * n_expert;
    for (int i = lane; i < n_expert; i += 32) wrow[i] = 0.f;
    if (tok >= n_rows) {
        if (lane == 0) shared_gate[tok] = 0.f;
        for (int j = lane; j < n_used; j += 32) route_idx[tok * n_used + j] = -1;
        return;
    }
    const float* x = logits + (uint64_t)tok * ld;
    float mx = -INFINITY;
    bool bad = false;
    for (int i = lane; i <= n_expert; i += 32) {   // the shared expert's gate logit (index n_expert) included
        const float v = x[i];
        bad |= !isfinite(v);
        if (i < n_expert) mx = fmaxf(mx, v);
    }
    if (__any_sync(0xffffffffu, bad)) {
        // route status NONFINITE (kernels/moe.metal:355-360): the row routes nowhere and the error word poisons the session
        if (lane == 0) {
            atomicCAS(err, 0, DEV_ERR_NONFINITE);
            shared_gate[tok] = 0.f;
        }
        for (int j = lane; j < n_used; j += 32) route_idx[tok * n_used + j] = -1;
        return;
    }
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

__global__ void __launch_bounds__(32) moe_route_kernel(const float* logits, int ld, int n_expert, int n_used, int n_rows,
                                                       float* route_w, float* shared_gate,
                                                       int32_t* route_idx, int* err) {
    pdl_prologue();
    __shared__ float p[MOE_MAX_EXPERTS];
    moe_route_row(p, blockIdx.x, threadIdx.x, logits, ld, n_expert, n_used, n_rows, route_w, shared_gate, route_idx, err);
}

dfl_status launch_moe_route(cudaStream_t st, const float* logits, int ld, int n_expert, int n_used, int n_rows, float* route_w,
                            float* shared_gate, int32_t* route_idx, int* err) {
    if (n_expert < 1 || n_expert > MOE_MAX_EXPERTS || n_used < 1 || n_used > 32 || n_used > n_expert)
        return fail(DFL_ERR_UNSUPPORTED, "moe_route: expert_count must be in [1, 1024] and expert_used_count in [1, 32]");
    launch_k(moe_route_kernel, dim3(MAX_ROWS), dim3(32), 0, st, logits, ld, n_expert, n_used, n_rows, route_w, shared_gate, route_idx, err);
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

// ---- the row tiles of the gate|up matrix that belong to chosen experts ------------------------------------------------
// The gate|up matrix of a layer is [gate of every local expert | shared gate | up of every local expert | shared up],
// T row tiles per expert and Ts per shared block.  An expert is active when any row of the block routes to it; the
// list holds the tiles of the active experts and of the shared expert, so the GEMM streams only those.  It is padded
// by repetition up to min_tiles (a repeated tile is computed twice with the same result), which keeps every CTA of the
// fixed launch geometry busy with at least one tile.
struct MoeListArgs {
    int n_expert, e0, n_local, T, Ts, min_tiles;
    int32_t *tile_map, *n_tiles;
    int KB, min_kb;
    int32_t *kb_map, *n_kb;
    int kc, down_tiles, max_splits, n_sm;
};
__device__ __forceinline__ void moe_build_lists(const float* route_w, const MoeListArgs a) {
    const int n_expert = a.n_expert, e0 = a.e0, n_local = a.n_local, T = a.T, Ts = a.Ts, min_tiles = a.min_tiles, KB = a.KB, min_kb = a.min_kb;
    const int kc = a.kc, down_tiles = a.down_tiles, max_splits = a.max_splits, n_sm = a.n_sm;
    int32_t *tile_map = a.tile_map, *n_tiles = a.n_tiles, *kb_map = a.kb_map, *n_kb = a.n_kb;
    __shared__ int warp_count[MOE_MAX_EXPERTS / 32];
    __shared__ int total_sh;
    const int e = threadIdx.x, warp = e >> 5, lane = e & 31;
    bool active = false;
    if (e < n_local) {
#pragma unroll
        for (int tok = 0; tok < MAX_ROWS; ++tok)   // independent loads (rows beyond the block are zero rows)
            active |= route_w[(uint64_t)tok * n_expert + e0 + e] != 0.f;
    }
    const uint32_t bal = __ballot_sync(0xffffffffu, active);
    if (lane == 0) warp_count[warp] = __popc(bal);
    __syncthreads();
    if (e == 0) {
        int run = 0;
        for (int w = 0; w < MOE_MAX_EXPERTS / 32; ++w) { const int c = warp_count[w]; warp_count[w] = run; run += c; }
        total_sh = run;
    }
    __syncthreads();
    const int n_act = total_sh, rank = warp_count[warp] + __popc(bal & ((1u << lane) - 1u));
    const int up_base = n_local * T + Ts, up_list = n_act * T + Ts, n = 2 * up_list;
    if (active)
        for (int j = 0; j < T; ++j) {
            tile_map[rank * T + j] = e * T + j;
            tile_map[up_list + rank * T + j] = up_base + e * T + j;
        }
    if (e < Ts) {
        tile_map[n_act * T + e] = n_local * T + e;
        tile_map[up_list + n_act * T + e] = up_base + n_local * T + e;
    }
    __syncthreads();
    for (int i = n + e; i < min_tiles; i += MOE_MAX_EXPERTS) tile_map[i] = n > 0 ? tile_map[i % n] : i;
    if (e == 0) *n_tiles = n > min_tiles ? n : min_tiles;
    // column blocks of the down matrix (KB per expert): the active experts' blocks first, then the others, whose
    // activations are zero - the list is cut after the active ones, but never below min_kb entries
    if (kb_map && e < n_local) {
        const int pos = active ? rank : n_act + (e - rank);
        for (int j = 0; j < KB; ++j) kb_map[pos * KB + j] = e * KB + j;
    }
    if (kb_map && e == 0) {
        const int want = n_act * KB, all = n_local * KB;
        const int len = want > min_kb ? want : (min_kb < all ? min_kb : all);
        n_kb[0] = len;
        // split geometry for this list length: enough splits to keep a CTA's blocks resident and to give every SM
        // work, as many CTAs per split as fit beside them; 0 = the launch's own geometry
        int s = 0, cps = 0;
        if (max_splits > 0) {
            s = (len + kc - 1) / kc;
            const int fill = (n_sm + down_tiles - 1) / down_tiles;
            if (s < fill) s = fill;
            if (s > max_splits) s = max_splits;
            if (s > len) s = len;
            cps = n_sm / s < down_tiles ? n_sm / s : down_tiles;
        }
        n_kb[1] = s;
        n_kb[2] = cps;
    }
}

__global__ void __launch_bounds__(MOE_MAX_EXPERTS) moe_tiles_kernel(const float* route_w, const MoeListArgs a) {
    pdl_prologue();
    moe_build_lists(route_w, a);
}
// routing of the block's rows (warps 0-15, one row each) and the lists in one launch
__global__ void __launch_bounds__(MOE_MAX_EXPERTS) moe_route_lists_kernel(const float* logits, int ld, int n_used, int n_rows, float* route_w,
                                                                          float* shared_gate, int32_t* route_idx, int* err, const MoeListArgs a) {
    pdl_prologue();
    extern __shared__ float p_rows[];   // [16][n_expert]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp < MAX_ROWS) moe_route_row(p_rows + warp * a.n_expert, warp, lane, logits, ld, a.n_expert, n_used, n_rows, route_w, shared_gate, route_idx, err);
    __syncthreads();   // the rows' route weights (global, written by this CTA) are complete
    moe_build_lists(route_w, a);
}

static MoeListArgs moe_list_args(int n_expert, int e0, int n_local, int tiles_per_expert, int shared_tiles, int min_tiles, int32_t* tile_map,
                                 int32_t* n_tiles, int kb_per_expert, int min_kb, int32_t* kb_map, int32_t* n_kb, int kc, int down_tiles,
                                 int max_splits) {
    return MoeListArgs{n_expert, e0, n_local, tiles_per_expert, shared_tiles, min_tiles, tile_map, n_tiles, kb_per_expert, min_kb, kb_map, n_kb,
                       kc, down_tiles, max_splits, sm_count()};
}

dfl_status launch_moe_tiles(cudaStream_t st, const float* route_w, int n_rows, int n_expert, int e0, int n_local, int tiles_per_expert,
                            int shared_tiles, int min_tiles, int32_t* tile_map, int32_t* n_tiles, int kb_per_expert, int min_kb, int32_t* kb_map,
                            int32_t* n_kb, int kc, int down_tiles, int max_splits) {
    (void)n_rows;
    if (n_local > MOE_MAX_EXPERTS || shared_tiles > MOE_MAX_EXPERTS) return fail(DFL_ERR_UNSUPPORTED, "moe_tiles: too many experts");
    launch_k(moe_tiles_kernel, dim3(1), dim3(MOE_MAX_EXPERTS), 0, st, route_w,
              moe_list_args(n_expert, e0, n_local, tiles_per_expert, shared_tiles, min_tiles, tile_map, n_tiles, kb_per_expert, min_kb, kb_map, n_kb,
                            kc, down_tiles, max_splits));
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

// routing + lists in one launch when the rows' probability scratch fits the default shared-memory window
bool moe_route_lists_fused(int n_expert) { return (size_t)MAX_ROWS * n_expert * 4 <= 40 * 1024; }
dfl_status launch_moe_route_lists(cudaStream_t st, const float* logits, int ld, int n_expert, int n_used, int n_rows, float* route_w,
                                  float* shared_gate, int32_t* route_idx, int e0, int n_local, int tiles_per_expert, int shared_tiles,
                                  int min_tiles, int32_t* tile_map, int32_t* n_tiles, int kb_per_expert, int min_kb, int32_t* kb_map,
                                  int32_t* n_kb, int kc, int down_tiles, int max_splits, int* err) {
    if (n_expert < 1 || n_used < 1 || n_used > 32 || n_used > n_expert || !moe_route_lists_fused(n_expert) || n_local > MOE_MAX_EXPERTS ||
        shared_tiles > MOE_MAX_EXPERTS)
        return fail(DFL_ERR_UNSUPPORTED, "moe_route_lists: geometry");
    launch_k(moe_route_lists_kernel, dim3(1), dim3(MOE_MAX_EXPERTS), (size_t)MAX_ROWS * n_expert * 4, st, logits, ld, n_used, n_rows, route_w,
              shared_gate, route_idx, err,
              moe_list_args(n_expert, e0, n_local, tiles_per_expert, shared_tiles, min_tiles, tile_map, n_tiles, kb_per_expert, min_kb, kb_map, n_kb,
                            kc, down_tiles, max_splits));
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

}  // namespace dfl
