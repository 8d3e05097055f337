// Kernel body and launcher of the tensor-memory few-row GEMM; included by gemm_ts.cu only.
//
// CTA = one split (at most KC column blocks, activations resident) x every ctas_per_split-th
// row tile.  Its work is the sequence of entries e = (tile, column block); the weight stage of
// entry e travels through ring slot e % STAGES.  Two groups of eight unpacking warps take the
// entries alternately (group = e & 1), each with its own tensor-memory buffers, MMA-issuing
// thread and barriers, so that one group's unpacking overlaps the other's waits; the groups
// meet only at the end of a row tile, where group 1 hands its partial sums to group 0 through
// shared memory and group 0 writes the tile.
//
// Inside a group an entry is processed in PASSES passes of 64 tensor-memory columns (Q4_K/Q5_K:
// 128 weight columns per pass, Q6_K: 64, twice, as the even/odd scale parts); the two pass
// buffers alternate, eight MMAs per pass accumulate into the group's single accumulator, which
// the group reads back while it already holds the next entry's first pass in registers.
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

#ifdef DFL_TS_TRACE
// development build only: SM-clock timestamps of CTA 0, [role][slot]; role 0 = group-0 warp 0, 1 = group-1 warp 8,
// 2 = MMA thread 0, 3 = MMA thread 1, 4 = producer
__device__ long long g_ts_trace[5][512];
#define TS_TRACE(role, slot)                                                                         \
    do {                                                                                             \
        if (blockIdx.x == 0 && (slot) < 512) g_ts_trace[role][slot] = clock64();                       \
    } while (0)
#else
#define TS_TRACE(role, slot) do { } while (0)
#endif

constexpr int XBUF_BYTES = GROUP_THREADS * 8 * 4;   // one tile's partial sums of a group: 8 tokens per thread

template <int DT>
constexpr int smem_bytes() {
    return KC * ACTTS_CHUNK + Fmt<DT>::STAGES * Fmt<DT>::STAGE + 2 * XBUF_BYTES + 256;
}

// named barrier 1: start-up of the unpacking warps (every one of them reaches it unconditionally)
__device__ __forceinline__ void named_sync(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }

template <int DT>
__global__ void __launch_bounds__(THREADS, 1) gemm_ts_kernel(const Params p) {
    using F = Fmt<DT>;
    constexpr int STAGES = F::STAGES, PASSES = F::PASSES;
    constexpr int OFF_RING = KC * ACTTS_CHUNK;
    constexpr int OFF_XBUF = OFF_RING + STAGES * F::STAGE;
    constexpr int OFF_BAR = OFF_XBUF + 2 * XBUF_BYTES;
    static_assert(OFF_BAR + 256 <= 227 * 1024, "shared memory budget");
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* acts_res = smem;
    uint8_t* ring = smem + OFF_RING;
    float* xbuf = reinterpret_cast<float*>(smem + OFF_XBUF);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
    uint64_t* empty = full + STAGES;
    uint64_t* acts_bar = empty + STAGES;
    uint64_t* a_ready = acts_bar + 1;   // [group][buffer] a pass of unpacked weights is in tensor memory
    uint64_t* a_free = a_ready + 4;     // [group][buffer] the MMAs of that pass have completed
    uint64_t* x_full = a_free + 4;      // [tile & 1] group 1 has put its partial sums of the tile into the exchange buffer
    uint64_t* x_free = x_full + 2;      // [tile & 1] group 0 has read them
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
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], GROUP_WARPS);
        }
        mbar_init(acts_bar, 1);
        for (int i = 0; i < 4; ++i) {
            mbar_init(&a_ready[i], GROUP_WARPS);
            mbar_init(&a_free[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&x_full[i], GROUP_WARPS);
            mbar_init(&x_free[i], GROUP_WARPS);
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
            const uint64_t tile_stride = (uint64_t)p.kblocks * F::STAGE;
            const uint8_t* wbase = p.w;
            int pt = 0, pk = 0;
            bool ok = true;
            for (int e = 0; e < n_it; ++e) {
                const int s = e % STAGES;
                if (e >= STAGES) ok = mbar_wait_bounded(&empty[s], ((e / STAGES) - 1) & 1, p.err, DEV_ERR_WAIT_EMPTY);
                if (!ok) break;
                const int slot = c + pt * cps;
                const uint8_t* src = wbase + (uint64_t)(p.tile_map ? p.tile_map[slot] : slot) * tile_stride +
                                     (uint64_t)(p.kb_map ? p.kb_map[kb0 + pk] : kb0 + pk) * F::STAGE;
                mbar_arrive_expect_tx(&full[s], F::STAGE);
                bulk_g2s(ring + s * F::STAGE, src, F::STAGE, &full[s]);
                TS_TRACE(4, e);
                if (++pk == n_kb) { pk = 0; ++pt; }
                if (e == (STAGES < n_it ? STAGES : n_it) - 1) {
                    // the ring is primed with weights (independent of the previous kernel); now the activations
                    pdl_wait();
                    mbar_arrive_expect_tx(acts_bar, (uint32_t)n_kb * ACTTS_CHUNK);
                    for (int k = 0; k < n_kb; ++k)
                        bulk_g2s(acts_res + k * ACTTS_CHUNK, p.acts + (uint64_t)(p.kb_map ? p.kb_map[kb0 + k] : kb0 + k) * ACTTS_CHUNK, ACTTS_CHUNK, acts_bar);
                }
            }
            if (!ok) abort_flag = 1;
        }
    } else if (warp == MMA_WARP0 || warp == MMA_WARP1) {
        // ------------------------------ MMA issuer of one group ------------------------------
        // The whole warp walks the loop so that addresses and descriptors stay warp-uniform; one elected
        // lane issues the instructions.
        const int g = warp - MMA_WARP0;
        if (n_it > g) {
            constexpr uint32_t IDESC_MAIN = instr_desc(32), IDESC_MIN = instr_desc(48);
            bool ok = mbar_wait_bounded(acts_bar, 0, p.err, DEV_ERR_WAIT_FULL);
            ok = __all_sync(0xffffffffu, ok);
            const uint32_t acts_addr = smem_u32(acts_res);
            const uint32_t tm_g = tmem + g * TM_GROUP;
            uint32_t pc = 0;   // running pass count of this group
            for (int e = g; e < n_it && ok; e += 2) {
                const uint32_t chunk = acts_addr + (e % n_kb) * ACTTS_CHUNK;
#pragma unroll
                for (int ps = 0; ps < PASSES; ++ps, ++pc) {
                    const uint32_t b = pc & 1;
                    if (ok) {
                        ok = mbar_wait_bounded(&a_ready[2 * g + b], (pc >> 1) & 1, p.err, DEV_ERR_WAIT_FULL);
                        ok = __all_sync(0xffffffffu, ok);
                    }
                    if (ok) {
                        if (lane == 0) TS_TRACE(2 + g, 2 * pc);
                        fence_after_sync();
                        if (elect_one()) {
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                mma_ts(tm_g + TM_D + 32 * (j & 1), tm_g + TM_A + b * 64 + 8 * j,
                                       smem_desc(chunk + F::b_slice(ps, j) * 1024, 512, 128), IDESC_MAIN, (ps | (j >> 1)) ? 1u : 0u);
                            if (F::HAS_MIN && ps == PASSES - 1)   // every pass has stored its column of the min operand by now
                                mma_ts(tm_g + TM_DM, tm_g + TM_AM, smem_desc(chunk + TS_BMIN_OFF, 768, 128), IDESC_MIN, 0);
                            mma_commit(&a_free[2 * g + b]);
                        }
                        __syncwarp();
                        if (lane == 0) TS_TRACE(2 + g, 2 * pc + 1);
                    }
                }
            }
            if (!ok) abort_flag = 1;
        }
    } else if (warp < UNPACK_WARPS) {
        // ------------------------------ unpack + drain warps ------------------------------
        pdl_wait();
        if (threadIdx.x < 256) {
            // per-token output scale; 16 threads per token add the sum-of-squares partials in a fixed tree
            const int tok = threadIdx.x >> 4, part = threadIdx.x & 15;
            float ss = 0.f;
            if (p.sumsq)
                for (int q = part; q < p.n_sumsq; q += 16) ss += p.sumsq[q * MAX_ROWS + tok];
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (part == 0) tok_scale[tok] = p.sumsq ? p.out_scale * (1.0f / sqrtf(ss / p.norm_k + p.eps)) : p.out_scale;
        }
        named_sync(1, UNPACK_WARPS * 32);

        const int g = warp >> 3, q4 = warp & 3, kp2 = (warp >> 2) & 1;
        const int row = 32 * q4 + lane, gtid = threadIdx.x & (GROUP_THREADS - 1);
        const uint32_t tm_g = tmem + g * TM_GROUP + ((uint32_t)(32 * q4) << 16);
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        // K padding of the min-term operand (sub-block index 8..15): written once, never touched again
        if (F::HAS_MIN && kp2 == 0) tmem_st4(tm_g + TM_AM + 4, 0u, 0u, 0u, 0u);
        bool ok = true;
        uint32_t pc = 0;            // running pass count of this group
        int next_close = 0;         // next row tile this group has to close
        bool pending = false;       // an entry whose accumulator has not been read back yet
        int pend_tile = 0;
        bool pend_last = false;
        UnitScales pend_us{0.f, 0.f};

        // hand over (group 1) or finish (group 0) the partial sums of tile t
        auto close_tile = [&](int t) {
            float* xb = xbuf + (t & 1) * (XBUF_BYTES / 4) + gtid * 8;
            const uint32_t use = (uint32_t)t >> 1;   // how often this exchange buffer has been used before
            if (g == 1) {
                if (t >= 2) {
                    ok = mbar_wait_bounded(&x_free[t & 1], (use - 1) & 1, p.err, DEV_ERR_WAIT_EMPTY);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) return;
                }
                *reinterpret_cast<float4*>(xb) = make_float4(acc[0], acc[1], acc[2], acc[3]);
                *reinterpret_cast<float4*>(xb + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
                __syncwarp();
                if (lane == 0) mbar_arrive(&x_full[t & 1]);
            } else {
                ok = mbar_wait_bounded(&x_full[t & 1], use & 1, p.err, DEV_ERR_WAIT_FULL);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) return;
                const float4 o0 = *reinterpret_cast<const float4*>(xb), o1 = *reinterpret_cast<const float4*>(xb + 4);
                const float other[8] = {o0.x, o0.y, o0.z, o0.w, o1.x, o1.y, o1.z, o1.w};
                __syncwarp();
                if (lane == 0) mbar_arrive(&x_free[t & 1]);
                const int slot = c + t * cps;
                const uint32_t orow = (uint32_t)(p.tile_map ? p.tile_map[slot] : slot) * TILE_R + row;
                if (orow < p.n_out) {
                    float* dst = p.out + ((uint64_t)sp * MAX_ROWS + 8 * kp2) * p.ld_out + orow;
#pragma unroll
                    for (int j = 0; j < 8; ++j) dst[(uint64_t)j * p.ld_out] = (acc[j] + other[j]) * tok_scale[8 * kp2 + j];
                }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        };
        // read back the accumulator of the pending entry (its last pass was pass pc - 1), scale, add
        auto drain_pending = [&]() {
            const uint32_t lp = pc - 1;
            ok = mbar_wait_bounded(&a_free[2 * g + (lp & 1)], (lp >> 1) & 1, p.err, DEV_ERR_WAIT_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) return;
            fence_after_sync();
            {
                float v[16], t[8];
                tmem_ld16(tm_g + TM_D + 16 * kp2, v);        // even MMA steps
                wait_ld();
#pragma unroll
                for (int j = 0; j < 8; ++j) t[j] = v[2 * j] + v[2 * j + 1];
                tmem_ld16(tm_g + TM_D + 32 + 16 * kp2, v);   // odd MMA steps
                wait_ld();
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] = fmaf(pend_us.d, t[j] + (v[2 * j] + v[2 * j + 1]), acc[j]);
            }
            if (F::HAS_MIN) {
                float s0[8], s1[8], s2[8];   // 8 tokens x 3 planes, token j = flattened columns 3j .. 3j + 2
                tmem_ld8(tm_g + TM_DM + 24 * kp2, s0);
                tmem_ld8(tm_g + TM_DM + 24 * kp2 + 8, s1);
                tmem_ld8(tm_g + TM_DM + 24 * kp2 + 16, s2);
                wait_ld();
                auto col = [&](int i) { return i < 8 ? s0[i] : i < 16 ? s1[i - 8] : s2[i - 16]; };
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] = fmaf(-pend_us.dmin, (col(3 * j) + col(3 * j + 1)) + col(3 * j + 2), acc[j]);
            }
            fence_before_sync();
            pending = false;
            if (pend_last) {
                close_tile(pend_tile);   // every earlier tile was closed when this entry was started
                next_close = pend_tile + 1;
            }
        };

        for (int e = g; e < n_it && ok; e += 2) {
            const int s = e % STAGES, tile = e / n_kb;
            const bool tracer = (warp & 7) == 0 && lane == 0;
            if (tracer) TS_TRACE(g, 16 * (e >> 1));
            ok = mbar_wait_bounded(&full[s], (e / STAGES) & 1, p.err, DEV_ERR_WAIT_FULL);
            if (tracer) TS_TRACE(g, 16 * (e >> 1) + 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const uint8_t* st = ring + s * F::STAGE;
            UnitScales us{0.f, 0.f};
#pragma unroll
            for (int ps = 0; ps < PASSES; ++ps, ++pc) {
                uint32_t r[32], am[8];
                if (ok) {
                    F::unpack(st, ps, row, kp2, r, am, us);
                }
                if (tracer) TS_TRACE(g, 16 * (e >> 1) + 2 + 3 * ps);
                if (ok && ps == 0) {
                    if (pending) drain_pending();
                    if (tracer) TS_TRACE(g, 16 * (e >> 1) + 14);
                    // tiles in which this group had no entry carry no partial sums of its own
                    while (ok && next_close < tile) close_tile(next_close++);
                }
                const uint32_t b = pc & 1;
                // The pass buffer was last read by pass pc - 2.  If that pass belongs to the previous entry, the
                // read-back above (or, for this group's first entries, nothing) already waited for it.
                if (ok && ps >= 2) {
                    ok = mbar_wait_bounded(&a_free[2 * g + b], ((pc >> 1) - 1) & 1, p.err, DEV_ERR_WAIT_FULL);
                    ok = __all_sync(0xffffffffu, ok);
                    if (ok) fence_after_sync();
                }
                if (tracer) TS_TRACE(g, 16 * (e >> 1) + 3 + 3 * ps);
                if (ok) {
                    F::store(tm_g + TM_A + b * 64, kp2, r);
                    if (F::HAS_MIN) tmem_st1(tm_g + TM_AM + 2 * ps + kp2, am[0]);
                    wait_st();
                    fence_before_sync();
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(&a_ready[2 * g + b]);
                        if (ps == PASSES - 1) mbar_arrive(&empty[s]);
                    }
                    if (tracer) TS_TRACE(g, 16 * (e >> 1) + 4 + 3 * ps);
                }
            }
            if (!ok) break;
            pending = true;
            pend_tile = tile;
            pend_last = e + 2 >= (tile + 1) * n_kb;   // this group's last entry of the tile
            pend_us = us;
        }
        if (ok && pending) drain_pending();
        while (ok && next_close < n_my) close_tile(next_close++);
        if (!ok) {
            abort_flag = 1;
        }
    }

    fence_before_sync();
    __syncthreads();
    if (abort_flag && threadIdx.x == 0) {
        // Error word already set.  Give every copy this CTA armed a bounded chance to land before
        // the shared memory is released.
        for (int s = 0; s < STAGES; ++s) {
            uint32_t spins = 0;
            while (!mbar_try_wait(&full[s], 0) && !mbar_try_wait(&full[s], 1) && ++spins < (1u << 16)) __nanosleep(100);
        }
        uint32_t spins = 0;
        while (!mbar_try_wait(acts_bar, 0) && ++spins < (1u << 16)) __nanosleep(100);
    }
    __syncthreads();
    if (warp == MMA_WARP0) {
        fence_after_sync();
        tmem_free(tmem, TM_COLS);
    }
}

template <int DT>
static dfl_status launch_t(cudaStream_t st, const Params& p, int grid, bool pdl) {
    static bool attr_set[16] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 16 && !attr_set[dev]) {
        DFL_CUDA(cudaFuncSetAttribute(gemm_ts_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes<DT>()));
        attr_set[dev] = true;
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
    int cps = 148 / splits;
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
    if (ep.kb_map && ep.dynamic_splits && grid < 148) grid = 148;   // room for the geometry chosen on the device
    switch (m.dtype) {
        case DFL_Q4_K: return ts::launch_t<DFL_Q4_K>(st, p, grid, pdl);
        case DFL_Q5_K: return ts::launch_t<DFL_Q5_K>(st, p, grid, pdl);
        case DFL_Q6_K: return ts::launch_t<DFL_Q6_K>(st, p, grid, pdl);
        default: return fail(DFL_ERR_UNSUPPORTED, "gemm: weight dtype has no tensor-memory kernel");
    }
}

}  // namespace dfl

#ifdef DFL_TS_TRACE
extern "C" int dfl_ts_trace_read(long long* out) {
    return (int)cudaMemcpyFromSymbol(out, dfl::ts::g_ts_trace, sizeof(long long) * 5 * 512);
}
#endif
