// Shared host/device helpers for the sm_100a kernels: status plumbing, bounded
// mbarrier waits, bulk (TMA 1-D) copies, programmatic-dependent-launch hooks and
// warp reductions.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>
#include <cstdio>
#include <string>

#include "../../include/dflash_b200.h"

namespace dfl {

// ---- host-side error plumbing ---------------------------------------------
void set_error(const std::string& msg);
dfl_status fail(dfl_status st, const std::string& msg);
extern std::atomic<uint64_t> g_launches;
inline void count_launch(uint64_t n = 1) { g_launches.fetch_add(n, std::memory_order_relaxed); }

#define DFL_CUDA(call)                                                                         \
    do {                                                                                       \
        cudaError_t _e = (call);                                                               \
        if (_e != cudaSuccess)                                                                 \
            return ::dfl::fail(DFL_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(_e)); \
    } while (0)

#define DFL_CHECK(st_expr)                   \
    do {                                     \
        dfl_status _s = (st_expr);           \
        if (_s != DFL_OK) return _s;         \
    } while (0)

// Device-side error word values (first failure wins).
enum DevErr : int {
    DEV_OK = 0,
    DEV_ERR_WAIT_FULL = 1,    // consumer gave up waiting for a stage to arrive
    DEV_ERR_WAIT_EMPTY = 2,   // producer gave up waiting for a stage to drain
    DEV_ERR_WAIT_DRAIN = 3,   // exit path gave up waiting for copies in flight
    DEV_ERR_NONFINITE = 4,    // NaN / Inf met where a finite value is required
    DEV_ERR_OVERFLOW = 5,     // activation outside the fp16 operand range
    DEV_ERR_WAIT_FLAG = 6,    // the wait probe (dfl_session_probe_wait_timeout): a barrier nobody arrives at
    DEV_ERR_WAIT_PEER = 7     // expert-parallel combine: a peer's contribution did not arrive (or the watchdog said stop)
};

#ifdef __CUDACC__
// ---- device helpers -------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// The same with a suspend-time hint: the thread may sleep in hardware for up to `ns` nanoseconds and is woken when the
// phase completes, so a waiting warp takes no issue slots from the warps that do the work.
__device__ __forceinline__ bool mbar_try_wait_for(uint64_t* bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
        : "memory");
    return ok != 0;
}
// Bounded wait: every wait in these kernels gives up after a fixed number of polls (each may sleep up to a
// microsecond: about a second in all), records why in *err and returns false, so a lost copy or a logic error ends
// the kernel instead of hanging the GPU.
constexpr uint32_t kWaitPolls = 1u << 20;
constexpr uint32_t kWaitSleepNs = 1000;
__device__ __forceinline__ bool mbar_wait_limit(uint64_t* bar, uint32_t parity, int* err, int code, uint32_t polls) {
    if (mbar_try_wait(bar, parity)) return true;
    for (uint32_t it = 0; it < polls; ++it)
        if (mbar_try_wait_for(bar, parity, kWaitSleepNs)) return true;
    atomicCAS(err, 0, code);
    return false;
}
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, int* err, int code) {
    return mbar_wait_limit(bar, parity, err, code, kWaitPolls);
}
// The same bound for a hand-off that sits on a kernel's critical path: polls without a suspend hint first (a sleeping
// thread is not always woken the moment the phase completes), then falls back to the sleeping wait.
constexpr uint32_t kSpinPolls = 1u << 14;
__device__ __forceinline__ bool mbar_wait_spin(uint64_t* bar, uint32_t parity, int* err, int code) {
    for (uint32_t it = 0; it < kSpinPolls; ++it)
        if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_limit(bar, parity, err, code, kWaitPolls);
}
// 1-D bulk async copy global -> shared, completion counted on an mbarrier.
// Both addresses 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
// Programmatic dependent launch: wait for the grids this launch depends on /
// allow dependents to start their prologue.  Both are no-ops for plain launches.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#endif  // __CUDACC__

// Kernels of the decode path are launched with programmatic stream serialization: a kernel may be
// scheduled while its predecessor in the stream is still running; it calls pdl_wait() before its
// first global-memory access and pdl_launch_dependents() at its top, so that launch latency and
// block scheduling overlap the predecessor.  DFL_PDL=0 turns the attribute off.
// Number of SMs of the current device (cached per device): grids are sized from it.
int sm_count();
bool pdl_enabled();
#ifdef __CUDACC__
template <typename... KArgs, typename... Args>
inline cudaError_t launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
// first statements of every kernel launched through launch_k.  Such a kernel starts its life before its
// predecessor has finished writing, so inputs the predecessor produces must not be declared
// `const T* __restrict__` (that licenses non-coherent read-only-cache loads, which may return stale lines);
// only genuinely immutable inputs (weights) keep the qualifier.
__device__ __forceinline__ void pdl_prologue() {
    pdl_launch_dependents();
    pdl_wait();
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Total-order key of an f32 (ascending): matches f32::total_cmp for non-NaN values.
__device__ __forceinline__ int32_t total_order_key(float f) {
    int32_t b = __float_as_int(f);
    return b < 0 ? (b ^ 0x7fffffff) : b;
}
#endif  // __CUDACC__

}  // namespace dfl
