// Row argmax + runner-up gap over device-resident logits, for callers that must not allocate.
//
// Same result as the argmax of the verify step (total order, lowest index on ties, NaN reported as
// ~index), but the per-row partial results live in a fixed array inside the loaded module instead
// of a cudaMalloc'ed buffer, the inputs and outputs are the caller's own device buffers, and the
// call only enqueues two kernels on the caller's stream.  Nothing here allocates, frees or
// synchronises.
#include <mutex>

#include "tiles.cuh"

namespace dfl {
dfl_status use_device(int device);
namespace {

constexpr int STATIC_MAX_ROWS = MAX_ROWS;       // 16 rows: one speculative block
constexpr int STATIC_PARTS = ARGMAX_PARTS;      // 64 column ranges per row
constexpr int STATIC_MAX_DEVICES = 64;

struct Best2 {
    int32_t k1, i1, k2, pad;  // total-order keys of best / runner-up, index of best
};

// 16 rows x 64 parts x 16 B = 16 KiB, shared by every call on the device.  Each call overwrites
// the slots of the rows it uses before reading them, so nothing in it has to start at zero.
static __device__ __align__(256) Best2 g_static_parts[STATIC_MAX_ROWS * STATIC_PARTS];

__device__ __forceinline__ Best2 best2_empty() { return Best2{INT32_MIN, INT32_MAX, INT32_MIN, 0}; }
__device__ __forceinline__ void best2_push(Best2& a, int32_t key, int32_t idx) {
    if (key > a.k1 || (key == a.k1 && idx < a.i1)) {
        a.k2 = a.k1;
        a.k1 = key;
        a.i1 = idx;
    } else if (key > a.k2) {
        a.k2 = key;
    }
}
__device__ __forceinline__ void best2_merge(Best2& a, const Best2& b) {
    if (b.k1 > a.k1 || (b.k1 == a.k1 && b.i1 < a.i1)) {
        a.k2 = a.k1 > b.k2 ? a.k1 : b.k2;
        a.k1 = b.k1;
        a.i1 = b.i1;
    } else {
        a.k2 = b.k1 > a.k2 ? b.k1 : a.k2;
    }
}
__device__ __forceinline__ Best2 best2_block(Best2 a) {
    __shared__ Best2 sh[32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best2 b;
        b.k1 = __shfl_xor_sync(0xffffffffu, a.k1, o);
        b.i1 = __shfl_xor_sync(0xffffffffu, a.i1, o);
        b.k2 = __shfl_xor_sync(0xffffffffu, a.k2, o);
        best2_merge(a, b);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    if (lane == 0) sh[warp] = a;
    __syncthreads();
    if (warp == 0) {
        a = lane < nw ? sh[lane] : best2_empty();
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            Best2 b;
            b.k1 = __shfl_xor_sync(0xffffffffu, a.k1, o);
            b.i1 = __shfl_xor_sync(0xffffffffu, a.i1, o);
            b.k2 = __shfl_xor_sync(0xffffffffu, a.k2, o);
            best2_merge(a, b);
        }
    }
    return a;
}
__device__ __forceinline__ float key_as_float(int32_t k) { return __int_as_float(k < 0 ? (k ^ 0x7fffffff) : k); }

// grid (64 parts, rows), block 256: best two of one column range of one row
__global__ void __launch_bounds__(256) argmax_static_part_kernel(const float* __restrict__ logits, uint64_t vocab, uint64_t ld,
                                                                 Best2* __restrict__ parts) {
    const int row = blockIdx.y, part = blockIdx.x;
    const uint64_t per = (vocab + STATIC_PARTS - 1) / STATIC_PARTS;
    const uint64_t lo = part * per, hi = lo + per < vocab ? lo + per : vocab;
    Best2 a = best2_empty();
    for (uint64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float v = logits[row * ld + i];
        best2_push(a, (v != v) ? INT32_MAX : total_order_key(v), (int32_t)i);
    }
    a = best2_block(a);
    if (threadIdx.x == 0) parts[row * STATIC_PARTS + part] = a;
}

// grid rows, block 64: merge the 64 parts of a row
__global__ void __launch_bounds__(64) argmax_static_final_kernel(const Best2* __restrict__ parts, int32_t* __restrict__ argmax,
                                                                 float* __restrict__ gap) {
    const int row = blockIdx.x;
    Best2 a = parts[row * STATIC_PARTS + threadIdx.x];
    a = best2_block(a);
    if (threadIdx.x == 0) {
        if (a.k1 == INT32_MAX) {
            argmax[row] = ~a.i1;
            gap[row] = 0.f;
        } else {
            argmax[row] = a.i1;
            gap[row] = a.k2 == INT32_MIN ? 0.f : key_as_float(a.k1) - key_as_float(a.k2);
        }
    }
}

std::mutex g_setup_mu;
Best2* g_parts_addr[STATIC_MAX_DEVICES] = {};

// Device address of the static array on `device` (which must be current); looked up once per device.
dfl_status static_parts_address(int device, Best2** out) {
    if (device >= STATIC_MAX_DEVICES) return fail(DFL_ERR_BAD_ARG, "argmax_top2_static: device index beyond 63");
    std::lock_guard<std::mutex> lk(g_setup_mu);
    if (!g_parts_addr[device]) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_static_parts);
        if (e != cudaSuccess || !p) {
            cudaGetLastError();
            return fail(DFL_ERR_CUDA, std::string("argmax_top2_static: cudaGetSymbolAddress: ") + cudaGetErrorString(e));
        }
        g_parts_addr[device] = static_cast<Best2*>(p);
    }
    *out = g_parts_addr[device];
    return DFL_OK;
}

}  // namespace
}  // namespace dfl

extern "C" dfl_status dfl_argmax_top2_static(int32_t device, const float* logits_dev, int32_t n_rows, uint64_t vocab, uint64_t ld,
                                             int32_t* argmax_dev, float* gap_dev, void* stream) {
    using namespace dfl;
    if (!logits_dev || !argmax_dev || !gap_dev) return fail(DFL_ERR_BAD_ARG, "argmax_top2_static: null pointer");
    if (n_rows < 1 || vocab == 0 || ld < vocab || vocab > 0x7fffffffull)
        return fail(DFL_ERR_BAD_SHAPE, "argmax_top2_static: need n_rows >= 1, 1 <= vocab <= ld, vocab < 2^31");
    if (n_rows > STATIC_MAX_ROWS)
        return fail(DFL_ERR_BAD_SHAPE, "argmax_top2_static: " + std::to_string(n_rows) + " rows exceed the fixed scratch of " +
                                           std::to_string(STATIC_MAX_ROWS) + " rows; split the call or use dfl_argmax_top2");
    DFL_CHECK(use_device(device));
    Best2* parts = nullptr;
    DFL_CHECK(static_parts_address(device, &parts));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    argmax_static_part_kernel<<<dim3(STATIC_PARTS, (unsigned)n_rows), 256, 0, st>>>(logits_dev, vocab, ld, parts);
    argmax_static_final_kernel<<<(unsigned)n_rows, 64, 0, st>>>(parts, argmax_dev, gap_dev);
    count_launch(2);
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}
