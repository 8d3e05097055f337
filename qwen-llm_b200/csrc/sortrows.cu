// Row-wise stable sort of logits on the device, for the host sampler (crates/qwen-llm/src/sampling.rs:305-790 orders
// every row by descending logit, total order, ties by ascending token, before it builds the row's distribution in f64;
// that ordering is more than half of the host's work per row at a 151 936-token vocabulary).  The order is a pure
// function of the bits of the logits, so computing it here changes nothing the sampler draws: the host still does the
// f64 exponentials and sums, in the order given.
//
// Key = descending_bits(logit): ascending key order == descending total order of the f32 (the host sampler's own key).
// LSD radix sort, four passes of 8 bits, stable; a row is cut into tiles of 1024 elements, one warp per tile (the
// tile's keys and values sit in the warp's registers, so every load is in flight before the ranking starts):
//   histogram   per (row, tile): 256 counters in shared memory
//   scan        per row: for every digit value, an exclusive prefix over the tiles in tile order, on top of the
//               exclusive prefix over the digit values
//   scatter     per (row, tile): the warp walks its tile in element order, 32 elements per step; __match_any_sync groups
//               the lanes with the same digit, the rank inside the group plus the tile's running count for that digit
//               is the element's place - which keeps equal keys in their previous order (initially token order)
// The values carried are the token ids; the last pass writes them straight into the output.
#include "model.cuh"
#include "ops.cuh"

namespace dfl {

namespace {
constexpr int SORT_TILE = 1024, SORT_WARPS = 4, SORT_PER_LANE = SORT_TILE / 32;

__device__ __forceinline__ uint32_t descending_bits_dev(float f) {
    const uint32_t b = __float_as_uint(f);
    const uint32_t asc = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
    return ~asc;
}

// the keys of one tile, element lo + 32 j + lane in k[j] (all loads issued before any is used); idle slots get key 0
// (key, token) pairs travel together between the passes: one 8-byte store per element instead of two 4-byte ones
template <bool FIRST>
__device__ __forceinline__ void load_tile(const float* logits, const uint2* pairs, uint64_t row_off, uint32_t lo, uint32_t hi, int lane,
                                          uint32_t (&k)[SORT_PER_LANE], uint32_t (&v)[SORT_PER_LANE]) {
#pragma unroll
    for (int j = 0; j < SORT_PER_LANE; ++j) {
        const uint32_t i = lo + 32u * j + lane;
        k[j] = 0u;
        v[j] = i;
        if (i < hi) {
            if (FIRST) k[j] = descending_bits_dev(logits[row_off + i]);
            else { const uint2 p = pairs[row_off + i]; k[j] = p.x; v[j] = p.y; }
        }
    }
}

// grid (ceil(tiles / 4), rows), block 128: warp w of block b owns tile 4 b + w
template <bool FIRST>
__global__ void __launch_bounds__(SORT_WARPS * 32) sort_hist_kernel(const float* logits, const uint2* pairs, uint32_t n, uint64_t ld, int shift,
                                                                    int tiles, uint32_t* counts /* [rows][tiles][256] */) {
    pdl_prologue();
    __shared__ uint32_t h[SORT_WARPS][256];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, row = blockIdx.y;
    const int tile = blockIdx.x * SORT_WARPS + warp;
    for (int b = lane; b < 256; b += 32) h[warp][b] = 0;
    __syncwarp();
    if (tile < tiles) {
        const uint32_t lo = (uint32_t)tile * SORT_TILE, hi = lo + SORT_TILE < n ? lo + SORT_TILE : n;
        uint32_t k[SORT_PER_LANE], v[SORT_PER_LANE];
        load_tile<FIRST>(logits, pairs, (uint64_t)row * ld, lo, hi, lane, k, v);
#pragma unroll
        for (int j = 0; j < SORT_PER_LANE; ++j)
            if (lo + 32u * j + lane < hi) atomicAdd(&h[warp][(k[j] >> shift) & 255u], 1u);
        __syncwarp();
        for (int b = lane; b < 256; b += 32) counts[((uint64_t)row * tiles + tile) * 256 + b] = h[warp][b];
    }
}

// grid (rows), block 1024: thread (q, b) owns digit value b over the q-th quarter of the tiles.  counts[row][tile][b]
// becomes the place of the first element of tile `tile` with digit b: the elements of smaller digits, then those of
// digit b in earlier tiles.
__global__ void __launch_bounds__(1024) sort_scan_kernel(uint32_t* counts, int tiles) {
    pdl_prologue();
    __shared__ uint32_t part[4][256];
    __shared__ uint32_t base[256];
    __shared__ uint32_t warp_sum[8];
    const int b = threadIdx.x & 255, q = threadIdx.x >> 8, lane = threadIdx.x & 31, row = blockIdx.x;
    const int per = (tiles + 3) / 4, t0 = q * per, t1 = min(tiles, t0 + per);
    uint32_t* c = counts + (uint64_t)row * tiles * 256 + b;
    uint32_t sum = 0;
#pragma unroll 8
    for (int t = t0; t < t1; ++t) sum += c[(uint64_t)t * 256];
    part[q][b] = sum;
    __syncthreads();
    if (q == 0) {   // exclusive prefix of the 256 digit totals
        const uint32_t total = part[0][b] + part[1][b] + part[2][b] + part[3][b];
        uint32_t incl = total;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const uint32_t up = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += up;
        }
        if (lane == 31) warp_sum[b >> 5] = incl;
        base[b] = incl - total;
    }
    __syncthreads();
    uint32_t run = base[b];
    for (int w = 0; w < (b >> 5); ++w) run += warp_sum[w];
    for (int p = 0; p < q; ++p) run += part[p][b];
#pragma unroll 8
    for (int t = t0; t < t1; ++t) {
        const uint32_t v = c[(uint64_t)t * 256];
        c[(uint64_t)t * 256] = run;
        run += v;
    }
}

template <bool FIRST>
__global__ void __launch_bounds__(SORT_WARPS * 32) sort_scatter_kernel(const float* logits, const uint2* pairs_in, uint32_t n, uint64_t ld, int shift, int tiles,
                                                                       const uint32_t* offsets, uint2* pairs_out, uint32_t* order_out, uint64_t ld_out) {
    pdl_prologue();
    __shared__ uint32_t run[SORT_WARPS][256];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, row = blockIdx.y;
    const int tile = blockIdx.x * SORT_WARPS + warp;
    if (tile >= tiles) return;
    const uint32_t lo = (uint32_t)tile * SORT_TILE, hi = lo + SORT_TILE < n ? lo + SORT_TILE : n;
    const uint64_t in_off = (uint64_t)row * ld, out_off = (uint64_t)row * ld_out;
    uint32_t k[SORT_PER_LANE], v[SORT_PER_LANE];
    load_tile<FIRST>(logits, pairs_in, in_off, lo, hi, lane, k, v);
    for (int b = lane; b < 256; b += 32) run[warp][b] = offsets[((uint64_t)row * tiles + tile) * 256 + b];
    __syncwarp();
#pragma unroll
    for (int j = 0; j < SORT_PER_LANE; ++j) {   // the tile in element order, 32 elements per step
        const bool live = lo + 32u * j + lane < hi;
        const uint32_t digit = live ? (k[j] >> shift) & 255u : 256u + (uint32_t)lane;   // idle lanes match nobody
        const uint32_t same = __match_any_sync(0xffffffffu, digit);
        const uint32_t before = __popc(same & ((1u << lane) - 1u));
        uint32_t place = 0;
        if (live) place = run[warp][digit] + before;
        __syncwarp();
        if (live && before == 0) run[warp][digit] += __popc(same);   // the group's first lane advances the running count
        __syncwarp();
        if (live) {
            if (pairs_out) pairs_out[out_off + place] = make_uint2(k[j], v[j]);
            else order_out[out_off + place] = v[j];     // the last pass: only the tokens are wanted
        }
    }
}
}  // namespace

uint64_t sort_rows_scratch_bytes(int n_rows, uint64_t vocab) {
    const uint64_t tiles = (vocab + SORT_TILE - 1) / SORT_TILE;
    return (uint64_t)n_rows * (4 * vocab + 256 * tiles) * 4;   // pairs A, pairs B, counters
}

// order[r][0..vocab) = token ids of row r by descending logit (total order), ties by ascending token
dfl_status launch_sort_rows_desc(cudaStream_t st, const float* logits, int n_rows, uint64_t vocab, uint64_t ld, void* scratch, uint32_t* order) {
    if (n_rows < 1 || vocab == 0 || vocab > 0x7fffffffull) return fail(DFL_ERR_BAD_SHAPE, "sort_rows: shape");
    const uint32_t n = (uint32_t)vocab;
    const int tiles = (int)((vocab + SORT_TILE - 1) / SORT_TILE);
    uint2* pa = reinterpret_cast<uint2*>(scratch);
    uint2* pb = pa + (uint64_t)n_rows * vocab;
    uint32_t* counts = reinterpret_cast<uint32_t*>(pb + (uint64_t)n_rows * vocab);
    const dim3 grid((unsigned)((tiles + SORT_WARPS - 1) / SORT_WARPS), (unsigned)n_rows), block(SORT_WARPS * 32);
    // pass p reads the logits (p = 0) or the pairs of pass p - 1 and writes pairs, the fourth pass the tokens alone
    const uint2* p_in = nullptr;
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 8 * pass;
        uint2* p_out = pass == 3 ? nullptr : (pass & 1) ? pb : pa;
        const uint64_t ld_in = pass == 0 ? ld : vocab;
        if (pass == 0) launch_k(sort_hist_kernel<true>, dim3(grid), dim3(block), 0, st, logits, p_in, n, ld_in, shift, tiles, counts);
        else launch_k(sort_hist_kernel<false>, dim3(grid), dim3(block), 0, st, logits, p_in, n, ld_in, shift, tiles, counts);
        launch_k(sort_scan_kernel, dim3((unsigned)n_rows), dim3(1024), 0, st, counts, tiles);
        if (pass == 0) launch_k(sort_scatter_kernel<true>, dim3(grid), dim3(block), 0, st, logits, p_in, n, ld_in, shift, tiles, (const uint32_t*)counts, p_out, order, vocab);
        else launch_k(sort_scatter_kernel<false>, dim3(grid), dim3(block), 0, st, logits, p_in, n, ld_in, shift, tiles, (const uint32_t*)counts, p_out, order, vocab);
        p_in = p_out;
    }
    count_launch(12);
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

}  // namespace dfl

using namespace dfl;

extern "C" dfl_status dfl_sort_rows_desc(int32_t device, const float* logits_host, int32_t n_rows, uint64_t vocab, uint32_t* order_out) {
    if (!logits_host || !order_out) return fail(DFL_ERR_BAD_ARG, "sort_rows: null argument");
    if (n_rows < 1 || n_rows > 1024 || vocab == 0 || vocab > 0x7fffffffull) return fail(DFL_ERR_BAD_SHAPE, "sort_rows: shape");
    DFL_CHECK(use_device(device));
    float* x = nullptr;
    uint32_t* order = nullptr;
    void* sc = nullptr;
    auto cleanup = [&]() { cudaFree(x); cudaFree(order); cudaFree(sc); };
    if (cudaMalloc(&x, (size_t)n_rows * vocab * 4) != cudaSuccess || cudaMalloc(&order, (size_t)n_rows * vocab * 4) != cudaSuccess ||
        cudaMalloc(&sc, sort_rows_scratch_bytes(n_rows, vocab)) != cudaSuccess) {
        cleanup();
        return fail(DFL_ERR_OOM, "sort_rows: cudaMalloc failed");
    }
    cudaMemcpy(x, logits_host, (size_t)n_rows * vocab * 4, cudaMemcpyHostToDevice);
    dfl_status s = launch_sort_rows_desc(0, x, n_rows, vocab, vocab, sc, order);
    if (s == DFL_OK && cudaMemcpy(order_out, order, (size_t)n_rows * vocab * 4, cudaMemcpyDeviceToHost) != cudaSuccess)
        s = fail(DFL_ERR_CUDA, "sort_rows: copy back failed");
    cleanup();
    return s;
}
