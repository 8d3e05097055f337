// bf16 weights on the fifth-generation tensor cores: no unpacking at all.  Included by gemm_ts.cu only.
//
// The resident tile of a bf16 matrix is stored directly in the shared-memory operand layout of
// tcgen05.mma (K-major, no swizzle: core matrices of 8 rows x 8 columns = 128 contiguous bytes,
// the 16 row groups of a k-core 128 B apart, k-cores 2048 B apart), half a 256-column block
// (128 rows x 128 columns = 32 KiB) per ring slot.  A bulk copy lands it where the MMA reads it:
//   producer thread : weights global -> ring, activations of the CTA's column range once;
//   MMA thread      : eight MMAs (M 128, N 48, K 16) per slot, A = weights and B = activations both
//                     from shared memory, one accumulator per row tile for the CTA's whole column
//                     range; tcgen05.commit releases the slot and, after the last slot of a tile,
//                     hands the accumulator to the epilogue;
//   four epilogue warps : read the 48 accumulator columns of their row (16 tokens x 3 bf16 planes of
//                     the activations), add the planes, scale, write the split-K partial.
// Two accumulators alternate so that the epilogue of one tile overlaps the MMAs of the next.
#pragma once

namespace dfl {

constexpr int TSB_SLOT = 32768;          // 128 rows x 128 columns of bf16
constexpr int TSB_KC = 4;                // column blocks whose activations stay resident
constexpr int TSB_STAGES = 4;
constexpr int TSB_THREADS = 6 * 32;      // producer warp, MMA warp, four epilogue warps
constexpr uint32_t TSB_TM_COLS = 128;    // two 48-column accumulators (at 0 and 64)

__host__ __device__ inline int tsb_w_offset(int r, int k) {   // inside a 256-column stage: two slots of 128 columns
    const int slot = k >> 7, kk = k & 127;
    return slot * TSB_SLOT + (kk >> 3) * 2048 + (r >> 3) * 128 + (r & 7) * 16 + (kk & 7) * 2;
}

// one thread per (row, 8 consecutive columns)
__global__ void retile_tsb_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, uint64_t n_in, uint64_t n_out, int kblocks) {
    const uint64_t tile_id = blockIdx.x;
    const int kb = (int)(tile_id % kblocks);
    const uint64_t rt = tile_id / kblocks;
    uint8_t* stage = dst + tile_id * STAGE_B16;
    for (int idx = threadIdx.x; idx < TILE_R * 32; idx += blockDim.x) {
        const int r = idx >> 5, k8 = (idx & 31) * 8;
        const uint64_t row = rt * TILE_R + r;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row < n_out) v = *reinterpret_cast<const uint4*>(src + (row * n_in + (uint64_t)kb * TILE_K + k8) * 2);
        *reinterpret_cast<uint4*>(stage + tsb_w_offset(r, k8)) = v;
    }
}
__device__ float decode_tsb_elem(const uint8_t* stage, int r, int k) {
    const uint16_t bits = *reinterpret_cast<const uint16_t*>(stage + tsb_w_offset(r, k));
    return __uint_as_float((uint32_t)bits << 16);
}

// standalone activation packing: one CTA per 256-column block; thread = (token, 16 consecutive columns)
__global__ void prep_acts_tsb_kernel(const float* __restrict__ x, int ld, int n_rows, float pre_scale, uint8_t* __restrict__ acts) {
    const int kb = blockIdx.x, tok = threadIdx.x >> 4, seg = threadIdx.x & 15;
    uint8_t* chunk = acts + (uint64_t)kb * ACTTSB_CHUNK;
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) {
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (tok < n_rows) {
            const float4 q = *reinterpret_cast<const float4*>(x + (uint64_t)tok * ld + (uint64_t)kb * TILE_K + seg * 16 + 4 * q4);
            v[0] = q.x * pre_scale; v[1] = q.y * pre_scale; v[2] = q.z * pre_scale; v[3] = q.w * pre_scale;
        }
        pack_quad_tsb(chunk, tok, seg * 16 + 4 * q4, v);
    }
}

namespace ts {

struct ParamsB {
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

constexpr int tsb_smem_bytes() { return TSB_KC * ACTTSB_CHUNK + TSB_STAGES * TSB_SLOT + 256; }

// bf16 x bf16 -> f32, both K-major, M = 128
__host__ __device__ constexpr uint32_t instr_desc_bf16(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((128u >> 4) << 24);
}

__global__ void __launch_bounds__(TSB_THREADS, 1) gemm_tsb_kernel(const ParamsB p) {
    constexpr int OFF_RING = TSB_KC * ACTTSB_CHUNK;
    constexpr int OFF_BAR = OFF_RING + TSB_STAGES * TSB_SLOT;
    static_assert(OFF_BAR + 256 <= 227 * 1024, "shared memory budget");
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* acts_res = smem;
    uint8_t* ring = smem + OFF_RING;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
    uint64_t* empty = full + TSB_STAGES;
    uint64_t* acts_bar = empty + TSB_STAGES;
    uint64_t* d_full = acts_bar + 1;    // [2] a tile's accumulator is complete
    uint64_t* d_empty = d_full + 2;     // [2] the epilogue has read it
    __shared__ uint32_t tmem_slot;
    __shared__ float tok_scale[MAX_ROWS];
    __shared__ int abort_flag;

    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
    const int sp = blockIdx.x % p.splits, c = blockIdx.x / p.splits;
    const int kb0 = (int)((long long)sp * p.kblocks / p.splits), kb1 = (int)((long long)(sp + 1) * p.kblocks / p.splits);
    const int n_kb = kb1 - kb0;
    const int n_my = (p.row_tiles - c + p.ctas_per_split - 1) / p.ctas_per_split;
    const int n_slots_tile = 2 * n_kb;           // ring slots (half column blocks) per row tile
    const int n_it = n_my * n_slots_tile;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TSB_STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(acts_bar, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&d_full[i], 1);
            mbar_init(&d_empty[i], 4);
        }
        abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(&tmem_slot, TSB_TM_COLS);
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem = tmem_slot;
    pdl_launch_dependents();

    if (warp == 0) {
        // ------------------------------ bulk-copy producer ------------------------------
        if (lane == 0) {
            const uint64_t tile_stride = (uint64_t)p.kblocks * STAGE_B16;
            const uint8_t* wbase = p.w + (uint64_t)kb0 * STAGE_B16;
            int pt = 0, pk = 0;
            bool ok = true;
            for (int e = 0; e < n_it; ++e) {
                const int s = e % TSB_STAGES;
                if (e >= TSB_STAGES) ok = mbar_wait_bounded(&empty[s], ((e / TSB_STAGES) - 1) & 1, p.err, DEV_ERR_WAIT_EMPTY);
                if (!ok) break;
                const uint8_t* src = wbase + (uint64_t)(c + pt * p.ctas_per_split) * tile_stride + (uint64_t)pk * TSB_SLOT;
                mbar_arrive_expect_tx(&full[s], TSB_SLOT);
                bulk_g2s(ring + s * TSB_SLOT, src, TSB_SLOT, &full[s]);
                if (++pk == n_slots_tile) { pk = 0; ++pt; }
                if (e == (TSB_STAGES < n_it ? TSB_STAGES : n_it) - 1) {
                    pdl_wait();   // the weights above do not depend on the previous kernel, the activations do
                    mbar_arrive_expect_tx(acts_bar, (uint32_t)n_kb * ACTTSB_CHUNK);
                    for (int k = 0; k < n_kb; ++k)
                        bulk_g2s(acts_res + k * ACTTSB_CHUNK, p.acts + (uint64_t)(kb0 + k) * ACTTSB_CHUNK, ACTTSB_CHUNK, acts_bar);
                }
            }
            if (!ok) abort_flag = 1;
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (n_it > 0) {
            constexpr uint32_t IDESC = instr_desc_bf16(48);
            bool ok = mbar_wait_bounded(acts_bar, 0, p.err, DEV_ERR_WAIT_FULL);
            ok = __all_sync(0xffffffffu, ok);
            const uint32_t acts_addr = smem_u32(acts_res), ring_addr = smem_u32(ring);
            int e = 0;
            for (int t = 0; t < n_my && ok; ++t) {
                const int buf = t & 1;
                if (t >= 2) {
                    ok = mbar_wait_bounded(&d_empty[buf], ((t >> 1) - 1) & 1, p.err, DEV_ERR_WAIT_EMPTY);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    fence_after_sync();
                }
                for (int h = 0; h < n_slots_tile && ok; ++h, ++e) {
                    const int s = e % TSB_STAGES;
                    ok = mbar_wait_bounded(&full[s], (e / TSB_STAGES) & 1, p.err, DEV_ERR_WAIT_FULL);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    fence_after_sync();
                    if (elect_one()) {
                        const uint32_t a_base = ring_addr + s * TSB_SLOT;
                        const uint32_t b_base = acts_addr + (h >> 1) * ACTTSB_CHUNK + (h & 1) * (16 * 768);   // 128 columns = 16 k-cores
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            mma_ss(tmem + 64 * buf, smem_desc(a_base + j * 4096, 2048, 128), smem_desc(b_base + j * 1536, 768, 128), IDESC,
                                   (h | j) ? 1u : 0u);
                        mma_commit(&empty[s]);                                    // slot free once these MMAs have read it
                        if (h == n_slots_tile - 1) mma_commit(&d_full[buf]);      // accumulator of the tile complete
                    }
                    __syncwarp();
                }
            }
            if (!ok) abort_flag = 1;
        }
    } else {
        // ------------------------------ epilogue warps ------------------------------
        pdl_wait();
        const int q4 = warp & 3;               // warps 2..5 -> tensor-memory lane quarters 2, 3, 0, 1
        const int row = 32 * q4 + lane;
        if (threadIdx.x - 64 < MAX_ROWS) {
            const int tok = threadIdx.x - 64;
            float ss = 0.f;
            if (p.sumsq)
                for (int q = 0; q < p.n_sumsq; ++q) ss += p.sumsq[q * MAX_ROWS + tok];
            tok_scale[tok] = p.sumsq ? p.out_scale * (1.0f / sqrtf(ss / p.norm_k + p.eps)) : p.out_scale;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const uint32_t lane_base = tmem + ((uint32_t)(32 * q4) << 16);
        bool ok = true;
        for (int t = 0; t < n_my && ok; ++t) {
            const int buf = t & 1;
            ok = mbar_wait_bounded(&d_full[buf], (t >> 1) & 1, p.err, DEV_ERR_WAIT_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            fence_after_sync();
            float v0[16], v1[16], v2[16];
            tmem_ld16(lane_base + 64 * buf, v0);
            tmem_ld16(lane_base + 64 * buf + 16, v1);
            tmem_ld16(lane_base + 64 * buf + 32, v2);
            wait_ld();
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&d_empty[buf]);
            auto col = [&](int i) { return i < 16 ? v0[i] : i < 32 ? v1[i - 16] : v2[i - 32]; };
            const uint32_t orow = (uint32_t)(c + t * p.ctas_per_split) * TILE_R + row;
            if (orow < p.n_out) {
                float* dst = p.out + (uint64_t)sp * MAX_ROWS * p.ld_out + orow;
#pragma unroll
                for (int tok = 0; tok < MAX_ROWS; ++tok)
                    dst[(uint64_t)tok * p.ld_out] = ((col(3 * tok) + col(3 * tok + 1)) + col(3 * tok + 2)) * tok_scale[tok];
            }
        }
        if (!ok) abort_flag = 1;
    }

    fence_before_sync();
    __syncthreads();
    if (abort_flag && threadIdx.x == 0) {
        for (int s = 0; s < TSB_STAGES; ++s) {
            uint32_t spins = 0;
            while (!mbar_try_wait(&full[s], 0) && !mbar_try_wait(&full[s], 1) && ++spins < (1u << 16)) __nanosleep(100);
        }
        uint32_t spins = 0;
        while (!mbar_try_wait(acts_bar, 0) && ++spins < (1u << 16)) __nanosleep(100);
    }
    __syncthreads();
    if (warp == 1) {
        fence_after_sync();
        tmem_free(tmem, TSB_TM_COLS);
    }
}

}  // namespace ts

int gemm_tsb_choose_splits_multi(const int* row_tiles, int n_mats, int kblocks) {
    const int s_min = (kblocks + TSB_KC - 1) / TSB_KC;
    int s_max = kblocks < 24 ? kblocks : 24;
    if (s_max < s_min) s_max = s_min;
    int best = s_min;
    double best_cost = 1e30;
    for (int s = s_min; s <= s_max; ++s) {
        double cost = 0.0;
        for (int i = 0; i < n_mats; ++i) {
            const int tiles = row_tiles[i] > 0 ? row_tiles[i] : 1;
            int cps = sm_count() / s;
            if (cps < 1) cps = 1;
            if (cps > tiles) cps = tiles;
            const int rounds = (tiles + cps - 1) / cps;
            cost += 0.02 * s + 0.002 * s * tiles + rounds * ((double)((kblocks + s - 1) / s) + 0.15);
        }
        if (cost < best_cost) { best_cost = cost; best = s; }
    }
    return best;
}

dfl_status launch_gemm_tsb(cudaStream_t st, const QMatrix& m, const uint8_t* acts, float* out, int splits, const GemmEpilogue& ep,
                           int* dev_err, bool pdl, uint32_t ld_out) {
    if (splits < 1 || splits > m.kblocks) return fail(DFL_ERR_BAD_ARG, "gemm: bad split count");
    if ((m.kblocks + splits - 1) / splits > TSB_KC) return fail(DFL_ERR_BAD_ARG, "gemm: too few splits for the resident activation window");
    ts::ParamsB p;
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
    int cps = sm_count() / splits;
    if (cps < 1) cps = 1;
    if (cps > m.row_tiles) cps = m.row_tiles;
    p.ctas_per_split = cps;
    p.n_out = (uint32_t)m.n_out;
    p.ld_out = ld_out ? ld_out : (uint32_t)m.n_out;
    p.err = dev_err;
    static bool attr_set[16] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 16 && !attr_set[dev]) {
        DFL_CUDA(cudaFuncSetAttribute(ts::gemm_tsb_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ts::tsb_smem_bytes()));
        attr_set[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(cps * splits));
    cfg.blockDim = dim3(TSB_THREADS);
    cfg.dynamicSmemBytes = ts::tsb_smem_bytes();
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    DFL_CUDA(cudaLaunchKernelEx(&cfg, ts::gemm_tsb_kernel, p));
    count_launch();
    return DFL_OK;
}

dfl_status launch_prep_acts_tsb(cudaStream_t st, const float* x, int ld, int n_rows, uint64_t k, float pre_scale, uint8_t* acts) {
    if (k % TILE_K || n_rows < 0 || n_rows > MAX_ROWS) return fail(DFL_ERR_BAD_SHAPE, "prep_acts: shape");
    prep_acts_tsb_kernel<<<(unsigned)(k / TILE_K), 256, 0, st>>>(x, ld, n_rows, pre_scale, acts);
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

}  // namespace dfl
