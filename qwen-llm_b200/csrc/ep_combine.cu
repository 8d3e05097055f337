// Expert-parallel combine over peer memory: the end of a routed-expert block when its experts are split over the GPUs
// of one node.  Each rank sums its own split-K slices of the down projection (slice order, as reduce_partials does),
// stores the [16][H] result into slot `rank` of EVERY rank's receive buffer with plain peer stores over NVLink,
// publishes a per-CTA sequence flag with a system-scope release, and waits (bounded) for the same CTA's flag of every
// peer in its own buffer.  The layer's glue kernel then reads the receive buffer as `world` slices and adds them in
// rank order, so every rank continues from bit-identical values - the all-reduce is the push plus the sum the glue
// does anyway, with no library collective on the path.  The reference runs its routed experts on one device
// (crates/qwen-llm/src/metal_forward/moe.rs:349-751); the multi-GPU split is this library's own.
//
// Buffers are double buffered on the parity of the sequence number: a rank can be at most one combine ahead of a peer
// (its next wait needs that peer's next push), so slot parity p is never rewritten while a peer still reads it.  The
// wait also polls a host-mapped abort word that the host watchdog raises, so a pass whose peer never arrives ends
// when the watchdog says so instead of at the kernel's own (long) limit.
#include "model.cuh"

namespace dfl {

namespace {
constexpr uint32_t kPeerPolls = 1u << 23;   // x 500 ns of sleep: several seconds, far beyond any healthy combine

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
}  // namespace

__global__ void __launch_bounds__(256) ep_push_sum_kernel(const float* part, int splits, const int32_t* splits_dev, uint64_t n_out,
                                                          EpPeers peers, int rank, int world, uint32_t seq, int n_cta,
                                                          const volatile int* abort_host, int* err) {
    pdl_prologue();
    if (splits_dev) splits += *splits_dev;
    const uint32_t parity = seq & 1u;
    const uint64_t n4 = (uint64_t)MAX_ROWS * n_out / 4, i4 = (uint64_t)blockIdx.x * 256 + threadIdx.x;
    if (i4 < n4) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s0 = 0; s0 < splits; s0 += 4) {   // slice order; four loads in flight per round trip
            float4 t[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int s = s0 + u < splits ? s0 + u : splits - 1;
                t[u] = __ldcg(reinterpret_cast<const float4*>(part + (uint64_t)s * MAX_ROWS * n_out) + i4);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (s0 + u < splits) { v.x += t[u].x; v.y += t[u].y; v.z += t[u].z; v.w += t[u].w; }
        }
        const uint64_t slot = ((uint64_t)parity * world + rank) * n4;   // float4 index of this rank's slot
        for (int p = 0; p < world; ++p) reinterpret_cast<float4*>(peers.base[p])[slot + i4] = v;
    }
    __threadfence_system();
    __syncthreads();
    if ((int)threadIdx.x < world) {
        const int p = threadIdx.x;
        const uint64_t flag_row = (uint64_t)parity * world;
        uint32_t* theirs = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(peers.base[p]) + peers.flags_off) + (flag_row + rank) * n_cta + blockIdx.x;
        st_release_sys(theirs, seq);   // this CTA's share of my slot is in peer p's buffer
        const uint32_t* mine = reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint8_t*>(peers.base[rank]) + peers.flags_off) + (flag_row + p) * n_cta + blockIdx.x;
        bool ok = false;
        for (uint32_t it = 0; it < kPeerPolls; ++it) {
            if ((int32_t)(ld_acquire_sys(mine) - seq) >= 0) { ok = true; break; }
            if ((it & 255u) == 255u && abort_host && *abort_host) break;
            __nanosleep(it < 64 ? 20 : 500);
        }
        if (!ok) atomicCAS(err, 0, DEV_ERR_WAIT_PEER);
    }
}

dfl_status launch_ep_push_sum(cudaStream_t st, const float* part, int splits, const int32_t* splits_dev, uint64_t n_out, const EpPeers& peers,
                              int rank, int world, uint32_t seq, const int* abort_host_dev, int* err) {
    const int n_cta = ep_combine_ctas(n_out);
    launch_k(ep_push_sum_kernel, dim3((unsigned)n_cta), dim3(256), 0, st, part, splits, splits_dev, n_out, peers, rank, world, seq, n_cta,
              (const volatile int*)abort_host_dev, err);
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

}  // namespace dfl
