// Top-16 (id, value) pairs of every row of a [rows][n] f32 matrix, in descending order under the f32 total order with
// ties to the lower index (reference: kernel_topk16_f32, kernels/dflash2.metal:69-170; unfilled slots keep the
// reference's sentinel (-inf, id -1)).
//
// An element is one 64-bit key: the total-order key of the value in the high word, the complemented index in the low
// word, so "better" is an unsigned compare and the answer is the 16 largest keys of the row together with 16 sentinel
// keys - independent of how the row is split over warps.  A warp keeps its 16 best keys one per lane (lane j = j-th
// best); a batch of 32 new keys is compared with the 16th best by ballot, and the few that beat it are inserted with
// two shuffles each.  Stage 1: rows x slices CTAs of 8 warps stream the row and leave one 16-list per warp; stage 2:
// one CTA per row merges those lists the same way (eight warps, then one).
#include "model.cuh"

namespace dfl {

namespace {
constexpr int TOPK = 16;
constexpr int TOPK_SLICES = 16, TOPK_WARPS = 8;   // lists per row = 128
constexpr uint64_t TOPK_SENTINEL = 0x007FFFFF00000000ull;   // (-inf, index 0xFFFFFFFF)

__device__ __forceinline__ uint64_t topk_key(float v, uint32_t idx) {
    const int32_t bits = __float_as_int(v);
    const uint32_t key = (uint32_t)(bits ^ (int32_t)((uint32_t)(bits >> 31) >> 1)) ^ 0x80000000u;   // unsigned total order
    return (uint64_t)key << 32 | (uint32_t)~idx;
}
__device__ __forceinline__ void topk_unkey(uint64_t k, float& v, int32_t& idx) {
    const uint32_t key = (uint32_t)(k >> 32) ^ 0x80000000u;
    const int32_t s = (int32_t)key;
    v = __int_as_float(s ^ (int32_t)((uint32_t)(s >> 31) >> 1));
    idx = (int32_t)~(uint32_t)k;
}
// lanes 0..15 hold the list in `mine` (descending); every lane offers one key
__device__ __forceinline__ void topk_offer(uint64_t& mine, uint64_t key, int lane) {
    uint64_t thr = __shfl_sync(0xffffffffu, mine, TOPK - 1);
    uint32_t mask = __ballot_sync(0xffffffffu, key > thr);
    while (mask) {
        const int src = __ffs(mask) - 1;
        mask &= mask - 1;
        const uint64_t cand = __shfl_sync(0xffffffffu, key, src);
        const uint64_t up = __shfl_up_sync(0xffffffffu, mine, 1);
        if (cand > thr) {   // uniform: thr and cand are warp-wide values
            if (mine < cand) mine = (lane == 0 || up > cand) ? cand : up;
            thr = __shfl_sync(0xffffffffu, mine, TOPK - 1);
        }
    }
}
}  // namespace

__global__ void __launch_bounds__(TOPK_WARPS * 32) topk16_stage1_kernel(const float* x, uint64_t n, uint64_t ld, uint64_t* lists) {
    pdl_prologue();
    const int row = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t wg = blockIdx.x * TOPK_WARPS + warp, n_w = TOPK_SLICES * TOPK_WARPS;
    const float* xr = x + (uint64_t)row * ld;
    uint64_t mine = TOPK_SENTINEL;
    for (uint64_t base = (uint64_t)wg * 32; base < n; base += (uint64_t)n_w * 32 * 4) {
        uint64_t k[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const uint64_t i = base + (uint64_t)u * n_w * 32 + lane;
            k[u] = i < n ? topk_key(xr[i], (uint32_t)i) : 0ull;   // 0 is below every key and the sentinel
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) topk_offer(mine, k[u], lane);
    }
    if (lane < TOPK) lists[((uint64_t)row * n_w + wg) * TOPK + lane] = mine;
}

__global__ void __launch_bounds__(TOPK_WARPS * 32) topk16_stage2_kernel(const uint64_t* lists, int n_lists, int32_t* ids, float* vals) {
    pdl_prologue();
    __shared__ uint64_t merged[TOPK_WARPS * TOPK];
    const int row = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int per_warp = (n_lists + TOPK_WARPS - 1) / TOPK_WARPS * TOPK;   // keys per warp
    const int n_keys = n_lists * TOPK;
    const uint64_t* l = lists + (uint64_t)row * n_keys;
    uint64_t mine = TOPK_SENTINEL;
    for (int base = warp * per_warp; base < (warp + 1) * per_warp; base += 32) {
        const int i = base + lane;
        topk_offer(mine, i < (warp + 1) * per_warp && i < n_keys ? l[i] : 0ull, lane);
    }
    if (lane < TOPK) merged[warp * TOPK + lane] = mine;
    __syncthreads();
    if (warp != 0) return;
    mine = TOPK_SENTINEL;
    for (int base = 0; base < TOPK_WARPS * TOPK; base += 32) topk_offer(mine, merged[base + lane], lane);
    if (lane < TOPK) {
        float v;
        int32_t idx;
        topk_unkey(mine, v, idx);
        ids[row * TOPK + lane] = idx;
        vals[row * TOPK + lane] = v;
    }
}

uint64_t topk16_scratch_bytes(int n_rows) { return (uint64_t)n_rows * TOPK_SLICES * TOPK_WARPS * TOPK * 8; }

dfl_status launch_topk16(cudaStream_t st, const float* x, int n_rows, uint64_t n, uint64_t ld, int32_t* ids, float* vals, void* scratch) {
    if (n_rows < 1 || n == 0 || n >= 0xFFFFFFFFull) return fail(DFL_ERR_BAD_SHAPE, "topk16: shape");
    launch_k(topk16_stage1_kernel, dim3(TOPK_SLICES, (unsigned)n_rows), dim3(TOPK_WARPS * 32), 0, st, x, n, ld, (uint64_t*)scratch);
    launch_k(topk16_stage2_kernel, dim3((unsigned)n_rows), dim3(TOPK_WARPS * 32), 0, st, (const uint64_t*)scratch, TOPK_SLICES * TOPK_WARPS, ids, vals);
    count_launch(2);
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

}  // namespace dfl

using namespace dfl;

extern "C" dfl_status dfl_topk16(int32_t device, const float* x_host, int32_t n_rows, uint64_t n, int32_t* ids_out, float* vals_out) {
    if (!x_host || !ids_out || !vals_out) return fail(DFL_ERR_BAD_ARG, "topk16: null argument");
    if (n_rows < 1 || n_rows > 1024 || n == 0) return fail(DFL_ERR_BAD_SHAPE, "topk16: shape");
    DFL_CHECK(use_device(device));
    float *x = nullptr, *v = nullptr;
    int32_t* id = nullptr;
    void* sc = nullptr;
    auto cleanup = [&]() { cudaFree(x); cudaFree(v); cudaFree(id); cudaFree(sc); };
    if (cudaMalloc(&x, (size_t)n_rows * n * 4) != cudaSuccess || cudaMalloc(&v, (size_t)n_rows * 64) != cudaSuccess ||
        cudaMalloc(&id, (size_t)n_rows * 64) != cudaSuccess || cudaMalloc(&sc, topk16_scratch_bytes(n_rows)) != cudaSuccess) {
        cleanup();
        return fail(DFL_ERR_OOM, "topk16: cudaMalloc failed");
    }
    cudaMemcpy(x, x_host, (size_t)n_rows * n * 4, cudaMemcpyHostToDevice);
    dfl_status s = launch_topk16(0, x, n_rows, n, n, id, v, sc);
    if (s == DFL_OK) {
        cudaError_t e1 = cudaMemcpy(ids_out, id, (size_t)n_rows * 64, cudaMemcpyDeviceToHost);
        cudaError_t e2 = cudaMemcpy(vals_out, v, (size_t)n_rows * 64, cudaMemcpyDeviceToHost);
        if (e1 != cudaSuccess || e2 != cudaSuccess) s = fail(DFL_ERR_CUDA, "topk16: copy back failed");
    }
    cleanup();
    return s;
}
