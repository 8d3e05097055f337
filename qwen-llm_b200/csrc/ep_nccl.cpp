// Expert parallelism plumbing: NCCL loaded at run time (the library must import on machines without it)
// and the one collective the routed-expert block needs - an all-reduce of the block's [16][H] output
// over the ranks that hold disjoint expert ranges.  The reference runs its routed experts on one device
// (crates/qwen-llm/src/metal_forward/moe.rs:349-751); the multi-GPU split is this library's own.
//
// Host watchdog: a pass of an expert-parallel model does not block in cudaStreamSynchronize, where a peer that
// never joins the collective would hold the caller for ever.  It records an event behind the pass and polls it,
// asking the communicator for an asynchronous error between polls; on an error, or when the event has not
// completed within the limit, the communicator is aborted (which ends the collective's kernels on this rank), the
// stream drains, and the caller gets DFL_ERR_COLLECTIVE with the session poisoned and the model's communicator
// marked dead.  The polling loop (ep_watch_core) takes its three actions as callbacks, so that it is exercised on the
// host with scripted ones (dfl_ep_watchdog_selftest).
#include <dlfcn.h>

#include <chrono>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>

#include "model.cuh"

namespace dfl {

namespace {
struct NcclId { char internal[128]; };
using comm_t = void*;
struct NcclApi {
    int (*GetUniqueId)(NcclId*) = nullptr;
    int (*CommInitRank)(comm_t*, int, NcclId, int) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, comm_t, cudaStream_t) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, comm_t, cudaStream_t) = nullptr;
    int (*CommDestroy)(comm_t) = nullptr;
    int (*CommAbort)(comm_t) = nullptr;
    int (*CommGetAsyncError)(comm_t, int*) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    bool ok = false;
};
NcclApi g_nccl;
std::once_flag g_nccl_once;

void load_nccl() {
    const char* names[] = {getenv("DFL_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
    void* h = nullptr;
    for (const char* n : names) {
        if (!n) continue;
        h = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (h) break;
    }
    if (!h) return;
    g_nccl.GetUniqueId = reinterpret_cast<decltype(g_nccl.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
    g_nccl.CommInitRank = reinterpret_cast<decltype(g_nccl.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
    g_nccl.AllReduce = reinterpret_cast<decltype(g_nccl.AllReduce)>(dlsym(h, "ncclAllReduce"));
    g_nccl.AllGather = reinterpret_cast<decltype(g_nccl.AllGather)>(dlsym(h, "ncclAllGather"));
    g_nccl.CommDestroy = reinterpret_cast<decltype(g_nccl.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
    g_nccl.CommAbort = reinterpret_cast<decltype(g_nccl.CommAbort)>(dlsym(h, "ncclCommAbort"));
    g_nccl.CommGetAsyncError = reinterpret_cast<decltype(g_nccl.CommGetAsyncError)>(dlsym(h, "ncclCommGetAsyncError"));
    g_nccl.GetErrorString = reinterpret_cast<decltype(g_nccl.GetErrorString)>(dlsym(h, "ncclGetErrorString"));
    g_nccl.ok = g_nccl.GetUniqueId && g_nccl.CommInitRank && g_nccl.AllReduce && g_nccl.CommDestroy;
}
dfl_status need_nccl() {
    std::call_once(g_nccl_once, load_nccl);
    if (!g_nccl.ok) return fail(DFL_ERR_UNSUPPORTED, "expert parallelism needs libnccl.so.2 (set DFL_NCCL_LIB or import torch first)");
    return DFL_OK;
}
dfl_status nccl_fail(const char* what, int rc) {
    return fail(DFL_ERR_CUDA, std::string(what) + ": " + (g_nccl.GetErrorString ? g_nccl.GetErrorString(rc) : "NCCL error") + " (" +
                                  std::to_string(rc) + ")");
}
}  // namespace

dfl_status ep_unique_id(uint8_t* id_out) {
    DFL_CHECK(need_nccl());
    NcclId id;
    const int rc = g_nccl.GetUniqueId(&id);
    if (rc != 0) return nccl_fail("ncclGetUniqueId", rc);
    memcpy(id_out, id.internal, 128);
    return DFL_OK;
}
dfl_status ep_comm_create(int rank, int world, const uint8_t* id_bytes, void** comm_out) {
    DFL_CHECK(need_nccl());
    NcclId id;
    memcpy(id.internal, id_bytes, 128);
    comm_t c = nullptr;
    const int rc = g_nccl.CommInitRank(&c, world, id, rank);
    if (rc != 0) return nccl_fail("ncclCommInitRank", rc);
    *comm_out = c;
    return DFL_OK;
}
void ep_comm_destroy(void* comm, bool aborted) {
    if (comm && g_nccl.ok && !aborted) g_nccl.CommDestroy(comm);   // an aborted communicator has been released by the abort
}

// The watchdog's loop.  query(): 0 = the pass has completed, 1 = still running, anything else = a CUDA error.
// async_error(): 0 = none (ncclSuccess), 7 = a non-blocking operation still in progress (ncclInProgress), anything else
// = the communicator has failed.  Returns DFL_OK when the pass completed; otherwise calls abort() once, waits (bounded)
// for the pass to drain, and returns DFL_ERR_COLLECTIVE.
dfl_status ep_watch_core(const EpWatchHooks& h, uint32_t timeout_ms, uint32_t poll_us, bool* aborted) {
    using clock = std::chrono::steady_clock;
    const auto t0 = clock::now();
    auto last_async = t0;
    *aborted = false;
    std::string why;
    for (;;) {
        const int q = h.query();
        if (q == 0) return DFL_OK;
        if (q != 1) { why = "the pass failed with a CUDA error while a collective was in flight"; break; }
        const auto now = clock::now();
        if (now - last_async >= std::chrono::microseconds(500)) {
            last_async = now;
            const int e = h.async_error();
            if (e != 0 && e != 7) { why = "the communicator reported an asynchronous error (" + std::to_string(e) + ")"; break; }
        }
        if (now - t0 >= std::chrono::milliseconds(timeout_ms)) {
            why = "a collective did not complete within " + std::to_string(timeout_ms) + " ms (a peer is missing or stalled)";
            break;
        }
        if (poll_us) std::this_thread::sleep_for(std::chrono::microseconds(poll_us));
        else std::this_thread::yield();
    }
    h.abort();
    *aborted = true;
    // the abort ends the collective's kernels; give the rest of the pass a bounded time to drain
    const auto t1 = clock::now();
    while (h.query() == 1 && clock::now() - t1 < std::chrono::milliseconds(timeout_ms)) std::this_thread::sleep_for(std::chrono::microseconds(200));
    return fail(DFL_ERR_COLLECTIVE, "expert-parallel watchdog: " + why + "; communicator aborted");
}

// Exchanges the inter-process handles of every rank's exchange buffer over the communicator and maps the peers' buffers
// into this process (plain peer loads and stores over NVLink).
dfl_status ep_p2p_exchange(void* comm, int rank, int world, void* local, cudaStream_t st, void** peers_out) {
    if (!g_nccl.AllGather) return fail(DFL_ERR_UNSUPPORTED, "expert-parallel combine: this NCCL has no ncclAllGather");
    if (world > EP_MAX_WORLD) return fail(DFL_ERR_UNSUPPORTED, "expert-parallel combine: at most 8 ranks");
    cudaIpcMemHandle_t mine;
    DFL_CUDA(cudaIpcGetMemHandle(&mine, local));
    uint8_t* dev_all = nullptr;
    DFL_CUDA(cudaMalloc(&dev_all, (size_t)world * sizeof(mine)));
    std::vector<cudaIpcMemHandle_t> all((size_t)world);
    cudaError_t e = cudaMemcpyAsync(dev_all + (size_t)rank * sizeof(mine), &mine, sizeof(mine), cudaMemcpyHostToDevice, st);
    int rc = 0;
    if (e == cudaSuccess) rc = g_nccl.AllGather(dev_all + (size_t)rank * sizeof(mine), dev_all, sizeof(mine), /*ncclUint8*/ 1, comm, st);
    if (e == cudaSuccess && rc == 0) e = cudaMemcpyAsync(all.data(), dev_all, (size_t)world * sizeof(mine), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess && rc == 0) e = cudaStreamSynchronize(st);
    cudaFree(dev_all);
    if (rc != 0) return nccl_fail("ncclAllGather", rc);
    DFL_CUDA(e);
    for (int p = 0; p < world; ++p) {
        if (p == rank) { peers_out[p] = local; continue; }
        void* ptr = nullptr;
        e = cudaIpcOpenMemHandle(&ptr, all[(size_t)p], cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            for (int q = 0; q < p; ++q)
                if (q != rank) cudaIpcCloseMemHandle(peers_out[q]);
            return fail(DFL_ERR_CUDA, std::string("expert-parallel combine: cannot map a peer's exchange buffer: ") + cudaGetErrorString(e));
        }
        peers_out[p] = ptr;
    }
    return DFL_OK;
}
void ep_p2p_close(int rank, int world, void* const* peers) {
    for (int p = 0; p < world; ++p)
        if (p != rank && peers[p]) cudaIpcCloseMemHandle(peers[p]);
}
// Every rank has reached this point: a one-element all-reduce, waited for under the watchdog loop with its own short
// limit, so that a peer that has already gone does not hold the caller.  False when the peers did not answer.
bool ep_barrier_bounded(void* comm, cudaStream_t st, uint32_t timeout_ms) {
    if (!g_nccl.CommAbort || !g_nccl.CommGetAsyncError) return false;
    float* one = nullptr;
    cudaEvent_t ev = nullptr;
    if (cudaMalloc(&one, 4) != cudaSuccess) return false;
    if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) { cudaFree(one); return false; }
    cudaMemsetAsync(one, 0, 4, st);
    bool ok = g_nccl.AllReduce(one, one, 1, 7, 0, comm, st) == 0 && cudaEventRecord(ev, st) == cudaSuccess;
    if (ok) {
        EpWatchHooks h;
        h.query = [ev]() -> int {
            const cudaError_t e = cudaEventQuery(ev);
            return e == cudaSuccess ? 0 : e == cudaErrorNotReady ? 1 : 2;
        };
        h.async_error = [comm]() -> int {
            int e = 0;
            const int rc = g_nccl.CommGetAsyncError(comm, &e);
            return rc != 0 ? rc : e;
        };
        h.abort = [comm]() { g_nccl.CommAbort(comm); };
        bool aborted = false;
        ok = ep_watch_core(h, timeout_ms, 100, &aborted) == DFL_OK;
    }
    cudaEventDestroy(ev);
    if (ok) cudaFree(one);   // after an abort the allocation is left to the end of the process
    return ok;
}

uint32_t ep_watch_timeout_ms() {
    // DFL_EP_TIMEOUT_MS: how long a pass of an expert-parallel model may take before its communicator is aborted
    static const uint32_t ms = [] {
        const char* e = getenv("DFL_EP_TIMEOUT_MS");
        const long v = e ? atol(e) : 0;
        return (uint32_t)(v > 0 ? v : 30000);
    }();
    return ms;
}

dfl_status ep_watch_stream(void* comm, cudaStream_t st, cudaEvent_t ev, volatile int* abort_word, bool* aborted) {
    *aborted = false;
    if (!g_nccl.CommAbort || !g_nccl.CommGetAsyncError) {   // an NCCL without these entry points: plain blocking wait
        DFL_CUDA(cudaStreamSynchronize(st));
        return DFL_OK;
    }
    DFL_CUDA(cudaEventRecord(ev, st));
    EpWatchHooks h;
    h.query = [ev]() -> int {
        const cudaError_t e = cudaEventQuery(ev);
        return e == cudaSuccess ? 0 : e == cudaErrorNotReady ? 1 : 2;
    };
    h.async_error = [comm]() -> int {
        int e = 0;
        const int rc = g_nccl.CommGetAsyncError(comm, &e);
        return rc != 0 ? rc : e;
    };
    h.abort = [comm, abort_word]() {
        if (abort_word) *abort_word = 1;   // ends the waits of the peer-memory combine kernels
        g_nccl.CommAbort(comm);
    };
    return ep_watch_core(h, ep_watch_timeout_ms(), 20, aborted);
}
// in-place sum over the ranks, f32; every rank receives the same bits
dfl_status ep_all_reduce_sum(void* comm, float* buf, size_t count, cudaStream_t st) {
    const int rc = g_nccl.AllReduce(buf, buf, count, /*ncclFloat32*/ 7, /*ncclSum*/ 0, comm, st);
    if (rc != 0) return nccl_fail("ncclAllReduce", rc);
    return DFL_OK;
}

}  // namespace dfl

extern "C" dfl_status dfl_ep_watchdog_selftest(int32_t scenario, uint32_t after_polls, uint32_t timeout_ms, int32_t* aborted_out) {
    using namespace dfl;
    if (!aborted_out || scenario < 0 || scenario > 3 || timeout_ms == 0 || timeout_ms > 10000)
        return fail(DFL_ERR_BAD_ARG, "ep_watchdog_selftest: scenario in [0, 3], timeout in (0, 10000] ms");
    uint32_t polls = 0;
    int aborts = 0;
    bool drained = false;
    EpWatchHooks h;
    h.query = [&]() -> int {
        ++polls;
        if (drained) return 0;   // after the abort the pass drains
        if (scenario == 0 && polls > after_polls) return 0;
        if (scenario == 3 && polls > after_polls) return 2;
        return 1;
    };
    h.async_error = [&]() -> int { return scenario == 1 && polls >= after_polls ? 6 /* ncclRemoteError */ : polls & 1 ? 0 : 7; };
    h.abort = [&]() { ++aborts; drained = true; };
    bool aborted = false;
    const dfl_status st = ep_watch_core(h, timeout_ms, 50, &aborted);
    *aborted_out = aborts;
    if ((aborts == 1) != aborted) return fail(DFL_ERR_CUDA, "ep_watchdog_selftest: abort ran a different number of times than reported");
    return st;
}
