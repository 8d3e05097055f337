// Expert parallelism plumbing: NCCL loaded at run time (the library must import on machines without it)
// and the one collective the routed-expert block needs - an all-reduce of the block's [16][H] output
// over the ranks that hold disjoint expert ranges.  The reference runs its routed experts on one device
// (crates/qwen-llm/src/metal_forward/moe.rs:349-751); the multi-GPU split is this library's own.
#include <dlfcn.h>

#include <cstring>
#include <mutex>
#include <string>

#include "model.cuh"

namespace dfl {

namespace {
struct NcclId { char internal[128]; };
using comm_t = void*;
struct NcclApi {
    int (*GetUniqueId)(NcclId*) = nullptr;
    int (*CommInitRank)(comm_t*, int, NcclId, int) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, comm_t, cudaStream_t) = nullptr;
    int (*CommDestroy)(comm_t) = nullptr;
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
    g_nccl.CommDestroy = reinterpret_cast<decltype(g_nccl.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
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
void ep_comm_destroy(void* comm) {
    if (comm && g_nccl.ok) g_nccl.CommDestroy(comm);
}
// in-place sum over the ranks, f32; every rank receives the same bits
dfl_status ep_all_reduce_sum(void* comm, float* buf, size_t count, cudaStream_t st) {
    const int rc = g_nccl.AllReduce(buf, buf, count, /*ncclFloat32*/ 7, /*ncclSum*/ 0, comm, st);
    if (rc != 0) return nccl_fail("ncclAllReduce", rc);
    return DFL_OK;
}

}  // namespace dfl
