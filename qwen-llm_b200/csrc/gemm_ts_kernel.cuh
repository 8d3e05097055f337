// Kernel body and launcher of the tensor-memory few-row GEMM; included by gemm_ts.cu only.
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
};

template <int DT>
constexpr int smem_bytes() {
    return KC * ACTTS_CHUNK + Fmt<DT>::STAGES * Fmt<DT>::STAGE + 256;
}

template <int DT>
__global__ void __launch_bounds__(THREADS, 1) gemm_ts_kernel(const Params p) {
    using F = Fmt<DT>;
    constexpr int STAGES = F::STAGES, UNITS = F::UNITS;
    constexpr int OFF_RING = KC * ACTTS_CHUNK;
    constexpr int OFF_BAR = OFF_RING + STAGES * F::STAGE;
    static_assert(OFF_BAR + 256 <= 227 * 1024, "shared memory budget");
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* acts_res = smem;
    uint8_t* ring = smem + OFF_RING;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
    uint64_t* empty = full + STAGES;
    uint64_t* acts_bar = empty + STAGES;
    uint64_t* a_ready = acts_bar + 1;   // [2] the unpacked A operand of a unit is in tensor memory
    uint64_t* mma_done = a_ready + 2;   // [2] the unit's MMAs have completed
    __shared__ uint32_t tmem_slot;
    __shared__ float tok_scale[MAX_ROWS];
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sp = blockIdx.x % p.splits, c = blockIdx.x / p.splits;
    const int kb0 = (int)((long long)sp * p.kblocks / p.splits), kb1 = (int)((long long)(sp + 1) * p.kblocks / p.splits);
    const int n_kb = kb1 - kb0;
    const int n_my = (p.row_tiles - c + p.ctas_per_split - 1) / p.ctas_per_split;   // row tiles c, c + cps, ...
    const int n_it = n_my * n_kb;            // stages
    const int n_units = n_it * UNITS;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], UNPACK_WARPS);
        }
        mbar_init(acts_bar, 1);
        for (int a = 0; a < 2; ++a) {
            mbar_init(&a_ready[a], UNPACK_WARPS);
            mbar_init(&mma_done[a], 1);
        }
        abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == MMA_WARP) tmem_alloc(&tmem_slot, TM_COLS);
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem = tmem_slot;
    pdl_launch_dependents();

    if (warp == PRODUCER_WARP) {
        // ------------------------------ bulk-copy producer ------------------------------
        if (lane == 0) {
            const uint64_t tile_stride = (uint64_t)p.kblocks * F::STAGE;
            const uint8_t* wbase = p.w + (uint64_t)kb0 * F::STAGE;
            int pt = 0, pk = 0;
            bool ok = true;
            for (int it = 0; it < n_it && ok; ++it) {
                const int s = it % STAGES;
                if (it >= STAGES) ok = mbar_wait_bounded(&empty[s], ((it / STAGES) - 1) & 1, p.err, DEV_ERR_WAIT_EMPTY);
                if (!ok) break;
                const uint8_t* src = wbase + (uint64_t)(c + pt * p.ctas_per_split) * tile_stride + (uint64_t)pk * F::STAGE;
                mbar_arrive_expect_tx(&full[s], F::STAGE);
                bulk_g2s(ring + s * F::STAGE, src, F::STAGE, &full[s]);
                if (++pk == n_kb) { pk = 0; ++pt; }
                if (it == (STAGES < n_it ? STAGES : n_it) - 1) {
                    // the ring is primed with weights (independent of the previous kernel); now the activations
                    pdl_wait();
                    mbar_arrive_expect_tx(acts_bar, (uint32_t)n_kb * ACTTS_CHUNK);
                    for (int k = 0; k < n_kb; ++k)
                        bulk_g2s(acts_res + k * ACTTS_CHUNK, p.acts + (uint64_t)(kb0 + k) * ACTTS_CHUNK, ACTTS_CHUNK, acts_bar);
                }
            }
            if (!ok) abort_flag = 1;
        }
    } else if (warp == MMA_WARP) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0 && n_units > 0) {
            constexpr uint32_t IDESC_MAIN = instr_desc(32), IDESC_MIN = instr_desc(48);
            bool ok = mbar_wait_bounded(acts_bar, 0, p.err, DEV_ERR_WAIT_FULL);
            const uint32_t acts_addr = smem_u32(acts_res);
            int kb = 0, u = 0;
            for (int i = 0; i < n_units && ok; ++i) {
                const int a = i & 1;
                ok = mbar_wait_bounded(&a_ready[a], (i >> 1) & 1, p.err, DEV_ERR_WAIT_FULL);
                if (!ok) break;
                fence_after_sync();
                const uint32_t chunk = acts_addr + kb * ACTTS_CHUNK;
                const uint32_t a_col = tmem + TM_A + a * 128, d_col = tmem + TM_D + a * 32;
#ifndef DFL_TS_EXP_NOMMA
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const uint32_t bk = F::b_kstep(u, j);   // which 16-column slice of the block this step multiplies with
                    mma_ts(d_col, a_col + 8 * j, smem_desc(chunk + bk * 1024, 512, 128), IDESC_MAIN, F::accumulate(j));
                }
#endif
                if (F::HAS_MIN) mma_ts(tmem + TM_DM + a * 48, tmem + TM_AM + a * 8, smem_desc(chunk + TS_BMIN_OFF, 768, 128), IDESC_MIN, 0);
                mma_commit(&mma_done[a]);
                if (++u == UNITS) { u = 0; if (++kb == n_kb) kb = 0; }
            }
            if (!ok) abort_flag = 1;
        }
    } else {
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
        asm volatile("bar.sync 1, %0;" ::"n"(UNPACK_THREADS) : "memory");

        const int q4 = warp & 3, kp = warp >> 2;
        const int row = 32 * q4 + lane;
        const uint32_t lane_base = tmem + ((uint32_t)(32 * q4) << 16);
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        UnitScales us_even{0.f, 0.f}, us_odd{0.f, 0.f};
        int dkb = 0, du = 0, dtile = 0;   // column block / unit / tile of the next unit to drain
        bool ok = true;

        // read back unit `i` (accumulators of buffer i & 1), scale and add; write the tile out after its last unit
        auto drain = [&](int i) {
            const int a = i & 1;
            ok = mbar_wait_bounded(&mma_done[a], (i >> 1) & 1, p.err, DEV_ERR_WAIT_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) return;
            fence_after_sync();
            float v[8];
            tmem_ld8(lane_base + TM_D + a * 32 + 8 * kp, v);
            float s[3][4];
            if (F::HAS_MIN) {
#pragma unroll
                for (int j = 0; j < 3; ++j) tmem_ld4(lane_base + TM_DM + a * 48 + 12 * kp + 4 * j, s[j]);
            }
            wait_ld();
            const UnitScales us = a ? us_odd : us_even;
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[j] = fmaf(us.d, v[2 * j] + v[2 * j + 1], acc[j]);
            if (F::HAS_MIN) {
                // s[..] flattened = 12 columns: token j -> planes 3j, 3j + 1, 3j + 2
                const float* f = &s[0][0];
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[j] = fmaf(-us.dmin, (f[3 * j] + f[3 * j + 1]) + f[3 * j + 2], acc[j]);
            }
            if (++du == UNITS) {
                du = 0;
                if (++dkb == n_kb) {
                    dkb = 0;
                    const uint32_t orow = (uint32_t)(c + dtile * p.ctas_per_split) * TILE_R + row;
                    if (orow < p.n_out) {
                        float* dst = p.out + ((uint64_t)sp * MAX_ROWS + 4 * kp) * p.ld_out + orow;
#pragma unroll
                        for (int j = 0; j < 4; ++j) dst[(uint64_t)j * p.ld_out] = acc[j] * tok_scale[4 * kp + j];
                    }
                    acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
                    ++dtile;
                }
            }
        };

        int u = 0;
        for (int i = 0; i < n_units; ++i) {
            const int it = i / UNITS, s = it % STAGES, a = i & 1;
            if (u == 0) {
                ok = mbar_wait_bounded(&full[s], (it / STAGES) & 1, p.err, DEV_ERR_WAIT_FULL);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
            }
            uint32_t r[32], am[8];
            UnitScales us;
#ifndef DFL_TS_EXP_NOUNPACK
            F::unpack(ring + s * F::STAGE, u, row, kp, r, am, us);
#else
            us.d = us.dmin = 0.f;
#pragma unroll
            for (int q = 0; q < 32; ++q) r[q] = 0u;
#pragma unroll
            for (int q = 0; q < 8; ++q) am[q] = 0u;
#endif
            if (i >= 2) {
                drain(i - 2);
                if (!ok) break;
            }
            if (a) us_odd = us; else us_even = us;
#ifndef DFL_TS_EXP_NOSTORE
            F::store(lane_base + TM_A + a * 128, kp, r);
#endif
            if (F::HAS_MIN && kp == 0) tmem_st8(lane_base + TM_AM + a * 8, am);
            wait_st();
            fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&a_ready[a]);
                if (u == UNITS - 1) mbar_arrive(&empty[s]);
            }
            if (++u == UNITS) u = 0;
        }
        if (ok && n_units >= 2) drain(n_units - 2);
        if (ok && n_units >= 1) drain(n_units - 1);
        if (!ok) abort_flag = 1;
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
    if (warp == MMA_WARP) {
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
    const int s_min = (m.kblocks + ts::KC - 1) / ts::KC;
    int s_max = m.kblocks < 24 ? m.kblocks : 24;
    if (s_max < s_min) s_max = s_min;
    int best = s_min;
    double best_cost = 1e30;
    for (int s = s_min; s <= s_max; ++s) {
        const int cps = ts::ctas_per_split(tiles, s);
        const int rounds = (tiles + cps - 1) / cps;
        const double unit = (double)((m.kblocks + s - 1) / s) + 0.25;
        const double cost = rounds * unit + 3.0 + 0.05 * s;
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
    const int grid = p.ctas_per_split * splits;
    switch (m.dtype) {
        case DFL_Q4_K: return ts::launch_t<DFL_Q4_K>(st, p, grid, pdl);
        case DFL_Q5_K: return ts::launch_t<DFL_Q5_K>(st, p, grid, pdl);
        case DFL_Q6_K: return ts::launch_t<DFL_Q6_K>(st, p, grid, pdl);
        default: return fail(DFL_ERR_UNSUPPORTED, "gemm: weight dtype has no tensor-memory kernel");
    }
}

}  // namespace dfl
