// Kernel body and launcher of the tensor-memory few-row GEMM; included by gemm_ts.cu only.
//
// CTA = one split (at most KC column blocks, activations resident) x every ctas_per_split-th
// row tile.  Its work is the sequence of entries e = (tile, column block); the weight stage of
// entry e travels through ring slot e % STAGES.  The sixteen unpacking warps form two groups of
// eight that take the entries alternately (group = e & 1), each with its own A buffer,
// accumulators and barriers, so that one group's arithmetic fills the time the other spends
// storing to tensor memory and waiting.  A group unpacks an entry in HALVES steps of 64 A-buffer
// columns (Q4_K / Q5_K: two halves of 128 weight columns; Q6_K: four of 64, each written as the
// even / odd scale parts); the MMA warp issues eight MMAs per half as soon as it is stored.
//
//   producer thread     ring slot free?   -> bulk copy of the stage          -> full[slot]   (activations: a draining thread)
//   unpacking group g   full[slot]        -> registers -> a_free[g][half]?   -> tcgen05.st -> a_ready[g][half], empty[slot]
//   MMA warp (g, c)     a_ready[g][c], d_free[g]?    -> 8 tcgen05.mma (+ min) -> commit: a_free[g][c], d_ready[g]
//                       (c = half % 2: its MMAs accumulate into accumulator c of the group, so the order in which the
//                       two warps of a group reach the tensor pipe does not change a bit of the result)
//   4 draining warps    d_ready[g]        -> tcgen05.ld -> d_free[g]         -> scale, add; tile end: global store
//
// The super-block scales d / dmin of an entry travel from the unpacking threads to the draining
// thread of the same row through a four-slot shared-memory side buffer (slot = entry & 3).
#pragma once

namespace dfl {
namespace ts {

struct Params {
    const uint8_t* w;
    const uint8_t* acts;
    float* out;
    const float* sumsq;
    int n_sumsq;
    float norm_k, eps, out_scale;
    int kblocks, splits, row_tiles, ctas_per_split;
    uint32_t n_out, ld_out;
    int* err;
    const int32_t* tile_map;   // optional: row tiles to compute, and how many (device memory)
    const int32_t* n_tiles;
    const int32_t* kb_map;     // optional: column blocks to sum over, and how many (device memory)
    const int32_t* n_kb;
};

constexpr int SCL_BYTES = 4 * TILE_R * 8;   // four entries' {d, dmin} per row
constexpr int BAR_BYTES = 512;              // up to 64 mbarriers

template <int DT>
constexpr int smem_bytes() {
    return KC * ACTTS_CHUNK + Fmt<DT>::STAGES * Fmt<DT>::STAGE + SCL_BYTES + BAR_BYTES;
}

// named barrier among the draining warps only (every one of them reaches it unconditionally)
__device__ __forceinline__ void named_sync(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }

// The eight MMAs of half h = 2 h2 + C of an entry into one accumulator (the first of them overwrites it when the half is
// the accumulator's first of the entry).
template <class F, int C>
__device__ __forceinline__ void issue_half(int h2, uint32_t d, uint32_t a_buf, uint32_t b_lo, uint32_t b_hi, uint32_t idesc) {
#pragma unroll
    for (int hh = 0; hh < F::HALVES / 2; ++hh) {
        if (hh != h2) continue;
        constexpr int dummy = 0;
        (void)dummy;
        const int h = 2 * hh + C;
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
            if (hh == 0 && jj == 0) mma_ts<false>(d, a_buf + F::a_col(h, jj), b_lo + F::b_slice(h, jj) * 64u, b_hi, idesc);
            else mma_ts<true>(d, a_buf + F::a_col(h, jj), b_lo + F::b_slice(h, jj) * 64u, b_hi, idesc);
        }
    }
}

template <int DT>
__global__ void __launch_bounds__(THREADS, 1) gemm_ts_kernel(const Params p) {
    using F = Fmt<DT>;
    constexpr int STAGES = F::STAGES, HALVES = F::HALVES;
    constexpr int OFF_RING = KC * ACTTS_CHUNK;
    constexpr int OFF_SCL = OFF_RING + STAGES * F::STAGE;
    constexpr int OFF_BAR = OFF_SCL + SCL_BYTES;
    // "Stage landed" barriers.  A parity wait is only meaningful to a waiter that knows the phase before is over, i.e. to
    // the one party that waits on that barrier phase after phase.  With an even number of stages a ring slot always
    // serves the same unpacking group; with an odd number its uses alternate between the two groups, and a group that
    // ran ahead could take the other group's still outstanding copy for its own (copies complete out of order).  So with
    // an odd number every slot has one barrier per group, each used by that group's uses of the slot only.
    constexpr int FULL_SETS = (STAGES & 1) ? 2 : 1;
    static_assert(OFF_BAR + BAR_BYTES <= 227 * 1024, "shared memory budget");
    static_assert((FULL_SETS + 1) * STAGES + KC + 12 <= BAR_BYTES / 8, "barrier area");
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* acts_res = smem;
    uint8_t* ring = smem + OFF_RING;
    float2* scl = reinterpret_cast<float2*>(smem + OFF_SCL);   // [entry & 3][row] = {d, dmin}
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
    uint64_t* empty = full + FULL_SETS * STAGES;
    auto full_bar = [](uint64_t* f, int e, int s) { return f + ((STAGES & 1) ? (e & 1) * STAGES : 0) + s; };
    // use number of the barrier: every use of the slot (even), or every second one (odd: the group's own)
    auto full_parity = [](int e) { return (uint32_t)((STAGES & 1) ? ((e / STAGES) >> 1) : (e / STAGES)) & 1u; };
    uint64_t* acts_bar = empty + STAGES;  // [column block of the CTA's range] its activations have arrived
    uint64_t* a_ready = acts_bar + KC;    // [group][half buffer] a half of unpacked weights is in tensor memory
    uint64_t* a_free = a_ready + 4;       // [group][half buffer] the MMAs of that half have completed
    uint64_t* d_ready = a_free + 4;       // [group] every MMA of an entry has completed
    uint64_t* d_free = d_ready + 2;       // [group] the draining warps have read the accumulator back
    __shared__ uint32_t tmem_slot;
    __shared__ float tok_scale[MAX_ROWS];
    __shared__ int abort_flag;

    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;   // warp-uniform by construction
    int row_tiles = p.row_tiles, kblocks = p.kblocks, splits = p.splits, cps = p.ctas_per_split;
    if (p.tile_map || p.kb_map) {   // the lists come from the preceding kernel: nothing may be fetched before it is complete
        pdl_wait();
        if (p.tile_map) row_tiles = *p.n_tiles;
        if (p.kb_map) {
            kblocks = p.n_kb[0];
            if (p.n_kb[1] > 0) {   // the list's author also chose the split geometry for its length (the launch is the worst case)
                splits = p.n_kb[1];
                cps = p.n_kb[2];
            }
        }
    }
    if ((int)blockIdx.x >= splits * cps) return;   // nothing has been set up yet: a CTA beyond the geometry in use just leaves
    const int sp = blockIdx.x % splits, c = blockIdx.x / splits;
    const int kb0 = (int)((long long)sp * kblocks / splits), kb1 = (int)((long long)(sp + 1) * kblocks / splits);
    const int n_kb = kb1 - kb0;
    const int n_my = (row_tiles - c + cps - 1) / cps;   // row tiles c, c + cps, ... (of the list)
    const int n_it = n_my * n_kb;            // entries

    if (threadIdx.x == 0) {
        for (int s = 0; s < FULL_SETS * STAGES; ++s) mbar_init(&full[s], 1);
        for (int s = 0; s < STAGES; ++s) mbar_init(&empty[s], GROUP_WARPS);
        for (int k = 0; k < KC; ++k) mbar_init(&acts_bar[k], 1);
        for (int i = 0; i < 4; ++i) {
            mbar_init(&a_ready[i], GROUP_WARPS);
            mbar_init(&a_free[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&d_ready[i], 2);
            mbar_init(&d_free[i], DRAIN_WARPS);
        }

        abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == MMA_WARP0) tmem_alloc(&tmem_slot, TM_COLS);
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem = tmem_slot;
    pdl_launch_dependents();

    if (warp == PRODUCER_WARP) {
        // ------------------------------ bulk-copy producer ------------------------------
        if (lane == 0) {
            // weights do not depend on the previous kernel: the ring is filled without waiting for it.  The loop keeps
            // running slot / round / source counters so that issuing a stage is a handful of instructions.
            const uint64_t tile_stride = (uint64_t)p.kblocks * F::STAGE;
            const bool mapped = p.tile_map != nullptr || p.kb_map != nullptr;
            int pt = 0, pk = 0, s = 0;
            uint32_t round = 0;
            const uint8_t* src = p.w + (uint64_t)c * tile_stride + (uint64_t)kb0 * F::STAGE;   // tile c, first column block of the range
            bool ok = true;
            for (int e = 0; e < n_it; ++e) {
                if (round > 0) ok = mbar_wait_bounded(&empty[s], (round - 1) & 1, p.err, DEV_ERR_WAIT_EMPTY);
                if (!ok) break;
                if (mapped) {
                    const int slot = c + pt * cps;
                    src = p.w + (uint64_t)(p.tile_map ? p.tile_map[slot] : slot) * tile_stride +
                          (uint64_t)(p.kb_map ? p.kb_map[kb0 + pk] : kb0 + pk) * F::STAGE;
                }
                uint64_t* fb = full_bar(full, e, s);
                mbar_arrive_expect_tx(fb, F::STAGE);
                bulk_g2s(ring + s * F::STAGE, src, F::STAGE, fb);
                src += F::STAGE;
                if (++s == STAGES) { s = 0; ++round; }
                if (++pk == n_kb) {   // next row tile of this CTA: cps tiles further, back to the first column block
                    pk = 0;
                    ++pt;
                    src += (uint64_t)cps * tile_stride - (uint64_t)n_kb * F::STAGE;
                }
            }
            if (!ok) abort_flag = 1;
        }
    } else if (warp >= MMA_WARP0 && warp < MMA_WARP0 + MMA_WARPS) {
        // ------------------------------ MMA issuers ------------------------------
        // Warp (g, c) issues the halves h with h % 2 == c of group g's entries into accumulator c of that group.  The
        // whole warp walks the loop so that addresses and descriptors stay warp-uniform; one elected lane issues.
        constexpr uint32_t IDESC_MAIN = instr_desc(32), IDESC_MIN = instr_desc(48);
        const uint32_t g = (uint32_t)(warp - MMA_WARP0) >> 1, c = (uint32_t)(warp - MMA_WARP0) & 1u;
        bool ok = true;
        const uint32_t acts_addr = smem_u32(acts_res);
        const uint32_t a_buf = tmem + TM_A + g * TM_A_STRIDE, d_buf = tmem + TM_D + g * TM_D_STRIDE + 32 * c;
        uint32_t uses = 0;   // how often this warp's half buffer has been used
        int kb_e = (int)g % n_kb;   // e % n_kb, kept by addition
        const int kb_step = 2 % n_kb;
        for (int e = (int)g; e < n_it && ok; e += 2) {
            const uint32_t chunk = acts_addr + (uint32_t)kb_e * ACTTS_CHUNK;
            kb_e += kb_step;
            if (kb_e >= n_kb) kb_e -= n_kb;
            if (e < n_kb) {   // first row tile: the column block's activations may still be in flight
                ok = mbar_wait_bounded(&acts_bar[e], 0, p.err, DEV_ERR_WAIT_FULL);
                ok = __all_sync(0xffffffffu, ok);
            }
            if (ok && e >= 2) {   // the group's accumulators were last used by entry e - 2
                ok = mbar_wait_bounded(&d_free[g], (((uint32_t)e >> 1) - 1) & 1, p.err, DEV_ERR_WAIT_EMPTY);
                ok = __all_sync(0xffffffffu, ok);
            }
            // one descriptor per column block; a 16-column slice is 1024 bytes further = 64 in the address field (bits 0-13
            // of the low word, which cannot carry: shared-memory addresses stay below 256 KiB)
            const uint64_t bdesc = smem_desc(chunk, 512, 128), mdesc = smem_desc(chunk + TS_BMIN_OFF, 768, 128);
            const uint32_t b_lo = (uint32_t)bdesc, b_hi = (uint32_t)(bdesc >> 32);
#pragma unroll
            for (int h2 = 0; h2 < HALVES / 2; ++h2, ++uses) {
                const int h = 2 * h2 + (int)c;   // this warp's half; the unrolled code below needs it as a constant: see the switch on c
                if (ok) {
                    ok = mbar_wait_bounded(&a_ready[2 * g + c], uses & 1, p.err, DEV_ERR_WAIT_FULL);
                    ok = __all_sync(0xffffffffu, ok);
                }
                if (ok) {
                    fence_after_sync();
                    if (elect_one()) {
                        if (c == 0) issue_half<F, 0>(h2, d_buf, a_buf, b_lo, b_hi, IDESC_MAIN);
                        else issue_half<F, 1>(h2, d_buf, a_buf, b_lo, b_hi, IDESC_MAIN);
                        if (F::HAS_MIN && h == HALVES - 1)   // every half has stored its column of the min operand by now
                            mma_ts<false>(tmem + TM_DM + g * TM_DM_STRIDE, tmem + TM_AM + g * TM_AM_STRIDE, (uint32_t)mdesc, (uint32_t)(mdesc >> 32),
                                          IDESC_MIN);
                        mma_commit(&a_free[2 * g + c]);
                        if (h2 == HALVES / 2 - 1) mma_commit(&d_ready[g]);   // this warp's share of the entry; the barrier counts both warps
                    }
                    __syncwarp();
                }
            }
        }
        if (!ok) abort_flag = 1;
    } else if (warp < UNPACK_WARPS) {
        // ------------------------------ unpacking warps ------------------------------
        // They read weights only (shared memory filled by the producer), so they never wait for the previous kernel.
        const int g = warp >> 3, q4 = warp & 3, kp2 = (warp >> 2) & 1;
        const int row = 32 * q4 + lane;
        const uint32_t tm_l = tmem + ((uint32_t)(32 * q4) << 16);
        const uint32_t a_buf = tm_l + TM_A + g * TM_A_STRIDE, am_buf = tm_l + TM_AM + g * TM_AM_STRIDE;
        // K padding of the group's min-term operand (sub-block pairs 4..7): written once, never touched again
        if (F::HAS_MIN && kp2 == 0) tmem_st4(am_buf + 4, 0u, 0u, 0u, 0u);
        bool ok = true;
        uint32_t hc = 0;   // running half count of this group
        for (int e = g; e < n_it && ok; e += 2) {
            const int s = e % STAGES;
            ok = mbar_wait_bounded(full_bar(full, e, s), full_parity(e), p.err, DEV_ERR_WAIT_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const uint8_t* st = ring + s * F::STAGE;
            uint32_t am_keep[HALVES];
#pragma unroll
            for (int h = 0; h < HALVES; ++h, ++hc) {
                uint32_t r[32], am[8];
                UnitScales us{0.f, 0.f};
                if (ok) F::unpack(st, h, row, kp2, r, am, us);
                if (F::HAS_MIN && h < HALVES - 1) am_keep[h] = am[0];
                const uint32_t hb = hc & 1;
                if (ok && hc >= 2) {   // the half buffer was last read by the MMAs of the group's half hc - 2
                    ok = mbar_wait_bounded(&a_free[2 * g + hb], ((hc >> 1) - 1) & 1, p.err, DEV_ERR_WAIT_FULL);
                    ok = __all_sync(0xffffffffu, ok);
                    if (ok) fence_after_sync();
                }
                if (ok) {
                    F::store(a_buf, h, kp2, r);
                    if (F::HAS_MIN && h == HALVES - 1) {
                        // The min operand is read by the entry's last MMA, so it may only be replaced once the previous
                        // entry's last half has completed - which this half's wait has just established.
#pragma unroll
                        for (int hh = 0; hh < HALVES - 1; ++hh) tmem_st1(am_buf + F::min_col(hh, kp2), am_keep[hh]);
                        tmem_st1(am_buf + F::min_col(h, kp2), am[0]);
                    }
                    if (h == 0 && kp2 == 0) scl[(e & 3) * TILE_R + row] = make_float2(us.d, us.dmin);
                    wait_st();
                    fence_before_sync();
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(&a_ready[2 * g + hb]);   // releases this warp's tensor-memory and side-buffer writes
                        if (h == HALVES - 1) mbar_arrive(&empty[s]);
                    }
                }
            }
        }
        if (!ok) abort_flag = 1;
    } else {
        // ------------------------------ draining warps ------------------------------
        pdl_wait();
        const int dtid = threadIdx.x - DRAIN_WARP0 * 32;   // 0..127 = weight row of the tile = tensor-memory lane
        if (dtid == 0 && n_it > 0) {
            // the activations (the previous kernel's output), in the order of their first use, one barrier each: the
            // first MMA waits for one chunk only.  Issued here rather than by the producer, whose first iterations are
            // busy priming the weight ring.
            for (int k = 0; k < n_kb; ++k) {
                mbar_arrive_expect_tx(&acts_bar[k], ACTTS_CHUNK);
                bulk_g2s(acts_res + k * ACTTS_CHUNK, p.acts + (uint64_t)(p.kb_map ? p.kb_map[kb0 + k] : kb0 + k) * ACTTS_CHUNK, ACTTS_CHUNK, &acts_bar[k]);
            }
        }
        {
            // per-token output scale; 8 threads per token add the sum-of-squares partials in a fixed tree
            const int tok = dtid >> 3, part = dtid & 7;
            float ss = 0.f;
            if (p.sumsq)
                for (int q = part; q < p.n_sumsq; q += 8) ss += p.sumsq[q * MAX_ROWS + tok];
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (part == 0) tok_scale[tok] = p.sumsq ? p.out_scale * (1.0f / sqrtf(ss / p.norm_k + p.eps)) : p.out_scale;
        }
        named_sync(1, DRAIN_WARPS * 32);
        const int row = dtid;
        const uint32_t tm_l = tmem + ((uint32_t)(32 * (warp & 3)) << 16);
        float acc[MAX_ROWS];
#pragma unroll
        for (int j = 0; j < MAX_ROWS; ++j) acc[j] = 0.f;
        bool ok = true;
        int kb_e = 0, tile = 0;   // e % n_kb and e / n_kb, kept by addition
        for (int e = 0; e < n_it && ok; ++e) {
            const uint32_t a = (uint32_t)e & 1u;
            ok = mbar_wait_bounded(&d_ready[a], ((uint32_t)e >> 1) & 1, p.err, DEV_ERR_WAIT_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            fence_after_sync();
            const float2 sc = scl[(e & 3) * TILE_R + row];   // published before the a_ready arrival the MMAs waited for
            float t[MAX_ROWS], mn[MAX_ROWS];
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {   // tokens 8 hf .. 8 hf + 7
                float ve[16], vo[16];
                tmem_ld16(tm_l + TM_D + a * TM_D_STRIDE + 16 * hf, ve);        // even MMA steps: columns 2 tok + plane
                tmem_ld16(tm_l + TM_D + a * TM_D_STRIDE + 32 + 16 * hf, vo);   // odd MMA steps
                if (F::HAS_MIN) {
                    float s0[8], s1[8], s2[8];   // 8 tokens x 3 planes, token j = flattened columns 3j .. 3j + 2
                    tmem_ld8(tm_l + TM_DM + a * TM_DM_STRIDE + 24 * hf, s0);
                    tmem_ld8(tm_l + TM_DM + a * TM_DM_STRIDE + 24 * hf + 8, s1);
                    tmem_ld8(tm_l + TM_DM + a * TM_DM_STRIDE + 24 * hf + 16, s2);
                    wait_ld();
                    auto col = [&](int i) { return i < 8 ? s0[i] : i < 16 ? s1[i - 8] : s2[i - 16]; };
#pragma unroll
                    for (int j = 0; j < 8; ++j) mn[8 * hf + j] = (col(3 * j) + col(3 * j + 1)) + col(3 * j + 2);
                } else {
                    wait_ld();
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) t[8 * hf + j] = (ve[2 * j] + ve[2 * j + 1]) + (vo[2 * j] + vo[2 * j + 1]);
            }
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&d_free[a]);   // the accumulator may be overwritten
#pragma unroll
            for (int j = 0; j < MAX_ROWS; ++j) {
                acc[j] = fmaf(sc.x, t[j], acc[j]);
                if (F::HAS_MIN) acc[j] = fmaf(-sc.y, mn[j], acc[j]);
            }
            if (++kb_e == n_kb) {   // the tile's last column block: write the partial result
                kb_e = 0;
                const int slot = c + tile * cps;
                ++tile;
                const uint32_t orow = (uint32_t)(p.tile_map ? p.tile_map[slot] : slot) * TILE_R + row;
                if (orow < p.n_out) {
                    float* dst = p.out + (uint64_t)sp * MAX_ROWS * p.ld_out + orow;
#pragma unroll
                    for (int j = 0; j < MAX_ROWS; ++j) dst[(uint64_t)j * p.ld_out] = acc[j] * tok_scale[j];
                }
#pragma unroll
                for (int j = 0; j < MAX_ROWS; ++j) acc[j] = 0.f;
            }
        }
        if (!ok) abort_flag = 1;
    }

    fence_before_sync();
    __syncthreads();
    if (abort_flag && threadIdx.x == 0) {
        // Error word already set.  Give every copy this CTA armed a bounded chance to land before
        // the shared memory is released.
        for (int s = 0; s < FULL_SETS * STAGES; ++s) {
            uint32_t spins = 0;
            while (!mbar_try_wait(&full[s], 0) && !mbar_try_wait(&full[s], 1) && ++spins < (1u << 16)) __nanosleep(100);
        }
        for (int k = 0; k < (n_it > 0 ? (n_kb < KC ? n_kb : KC) : 0); ++k) {
            uint32_t spins = 0;
            while (!mbar_try_wait(&acts_bar[k], 0) && ++spins < (1u << 16)) __nanosleep(100);
        }
    }
    __syncthreads();
    if (warp == MMA_WARP0) {
        fence_after_sync();
        tmem_free(tmem, TM_COLS);
    }
}

template <int DT>
static dfl_status launch_t(cudaStream_t st, const Params& p, int grid, bool pdl) {
    static std::once_flag attr_once[16];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 16) {
        cudaError_t attr_err = cudaSuccess;
        std::call_once(attr_once[dev], [&] {
            attr_err = cudaFuncSetAttribute(gemm_ts_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes<DT>());
        });
        DFL_CUDA(attr_err);
    } else {
        DFL_CUDA(cudaFuncSetAttribute(gemm_ts_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes<DT>()));
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem_bytes<DT>();
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    DFL_CUDA(cudaLaunchKernelEx(&cfg, gemm_ts_kernel<DT>, p));
    count_launch();
    return DFL_OK;
}

static int ctas_per_split(int row_tiles, int splits) {
    int cps = sm_count() / splits;
    if (cps < 1) cps = 1;
    return cps < row_tiles ? cps : row_tiles;
}

}  // namespace ts

// Split count: every split must fit the resident activation window; beyond that, the count that
// minimises the longest CTA (rounds of row tiles x column blocks per split, plus a per-tile
// and a per-launch overhead measured in stage times).
int gemm_ts_choose_splits(const QMatrix& m) {
    const int tiles = m.row_tiles > 0 ? m.row_tiles : 1;
    return gemm_ts_choose_splits_multi(&tiles, 1, m.kblocks);
}
// CTAs per split of a launch over `row_tiles` row tiles (the least number of tiles a tile list must hold)
int gemm_ts_kc() { return ts::KC; }   // column blocks a CTA keeps resident
int gemm_ts_ctas_per_split(int row_tiles, int splits) { return ts::ctas_per_split(row_tiles, splits); }
// Several matrices that share their input and their partial buffer are launched one after the other
// with one common split count: minimise the sum of their longest-CTA times.
int gemm_ts_choose_splits_multi(const int* row_tiles, int n_mats, int kblocks) {
    const int s_min = (kblocks + ts::KC - 1) / ts::KC;
    int s_max = kblocks < 24 ? kblocks : 24;
    if (s_max < s_min) s_max = s_min;
    int best = s_min;
    double best_cost = 1e30;
    for (int s = s_min; s <= s_max; ++s) {
        double cost = 0.0;
        for (int i = 0; i < n_mats; ++i) {
            const int tiles = row_tiles[i] > 0 ? row_tiles[i] : 1;
            cost += 0.05 * s + 0.0054 * s * tiles;   // partial slices to write and to sum again
            const int cps = ts::ctas_per_split(tiles, s);
            const int rounds = (tiles + cps - 1) / cps;
            cost += rounds * ((double)((kblocks + s - 1) / s) + 0.25);
        }
        if (cost < best_cost) { best_cost = cost; best = s; }
    }
    return best;
}

dfl_status launch_gemm_ts(cudaStream_t st, const QMatrix& m, const uint8_t* acts, float* out, int splits, const GemmEpilogue& ep,
                          int* dev_err, bool pdl, uint32_t ld_out) {
    if (splits < 1 || splits > m.kblocks) return fail(DFL_ERR_BAD_ARG, "gemm: bad split count");
    if ((m.kblocks + splits - 1) / splits > ts::KC) return fail(DFL_ERR_BAD_ARG, "gemm: too few splits for the resident activation window");
    ts::Params p;
    p.w = m.tiles;
    p.acts = acts;
    p.out = out;
    p.sumsq = ep.sumsq;
    p.n_sumsq = ep.n_sumsq;
    p.norm_k = ep.norm_k;
    p.eps = ep.eps;
    p.out_scale = ep.out_scale;
    p.kblocks = m.kblocks;
    p.splits = splits;
    p.row_tiles = m.row_tiles;
    p.ctas_per_split = ts::ctas_per_split(m.row_tiles, splits);
    p.n_out = (uint32_t)m.n_out;
    p.ld_out = ld_out ? ld_out : (uint32_t)m.n_out;
    p.err = dev_err;
    p.tile_map = ep.tile_map;
    p.n_tiles = ep.n_tiles;
    p.kb_map = ep.kb_map;
    p.n_kb = ep.n_kb;
    int grid = p.ctas_per_split * splits;
    if (ep.kb_map && ep.dynamic_splits && grid < sm_count()) grid = sm_count();   // room for the geometry chosen on the device
    switch (m.dtype) {
        case DFL_Q4_K: return ts::launch_t<DFL_Q4_K>(st, p, grid, pdl);
        case DFL_Q5_K: return ts::launch_t<DFL_Q5_K>(st, p, grid, pdl);
        case DFL_Q6_K: return ts::launch_t<DFL_Q6_K>(st, p, grid, pdl);
        case DFL_Q8_0: return ts::launch_t<DFL_Q8_0>(st, p, grid, pdl);
        default: return fail(DFL_ERR_UNSUPPORTED, "gemm: weight dtype has no tensor-memory kernel");
    }
}

}  // namespace dfl
