// Verify attention over a long fp16 KV cache on the fifth-generation tensor cores (tcgen05 + tensor memory), for
// 128-wide heads in GQA groups of four (reference: kernel_attn_decode_* / attn_v4, kernels/attn_v4.metal:65-265; CPU
// oracle forward.rs:896-921).
//
// Cache layout ("tiled", sessions whose KV capacity makes the scan the dominant cost): per (128-position chunk, KV head)
// one 32 KiB K tile and one 32 KiB V tile, each already in the K-major, no-swizzle operand layout of tcgen05.mma
// (8 x 16-byte core matrices): K as B[n = key][k = dim], V as B[n = dim][k = key].  A tile is one bulk copy into shared
// memory and is consumed by the tensor cores as it lies; appending a position writes 16-byte pieces (K) and single
// halfs (V) into the last tile (attn_front_kernel).
//
// One CTA = one KV head x one span of `chunks_per_span` tiles; the 16 block rows x 4 query heads of the group are the
// 64 queries.  Tensor-memory lane r and lane r + 64 both hold query r & 63: the A operand of S = Q K^T is [Q; Q]
// (M = 128) with K = 256 - the f16 hi plane, then the lo plane of the pre-scaled queries, each against the K tile - so S
// is exact to ~2^-22 like the mma.sync kernel's.  The operand lives in tensor memory (written once per CTA with
// tcgen05.st), so shared memory only carries K and V tiles.  Every lane is one softmax thread: lanes 0-63 own keys 0-63
// of each tile for their query, lanes 64-127 keys 64-127 - two independent online-softmax states per query, each with
// its own running maximum, sum and output row.  P (f16; the lane's own half of the keys, zeros in the other half) is
// written over the scores it came from and is the A operand of O += P V, so each lane's output row only collects its
// own keys.  The output is rescaled only when a lane's maximum grows by more than 2^8 (its P values stay below 256; the
// record keeps the maximum that was used), which leaves the O accumulator in tensor memory untouched in nearly every
// step.  At the end each lane writes one [m, l, O[128]] record; attn_post_kernel merges the two records per span and the
// spans exactly as it merges the other kernels' records.  Span boundaries depend only on the session's KV capacity,
// never on the call.
//
// Warps 0-3: softmax / rescale / epilogue (thread = lane of tensor memory); warp 4: MMA issue (one elected lane) and
// tensor-memory allocation; warp 5: bulk copies of the tiles into a ring of six 32 KiB slots (K and V tiles alternate;
// a K slot is released when its S is complete, a V slot when its O += P V is).  Every wait is bounded and reports
// through the error word; a role that gave up raises a flag the others test, all of them leave through the common exit,
// and tensor memory is freed on every path.
#include <cuda_fp16.h>

#include <mutex>

#include "ops.cuh"
#include "tcgen05_prims.cuh"

namespace dfl {

namespace {
using namespace ts;

constexpr int T5_HD = 128, T5_GROUP = 4, T5_Q = MAX_ROWS * T5_GROUP;   // 64 queries per CTA
constexpr int T5_TILE = KV_TILE_KEYS * T5_HD * 2;                      // 32768 bytes: one K or V tile
constexpr int T5_SLOTS = 6;
constexpr int T5_QPITCH = T5_HD + 1;                                   // floats per staged query row (odd: a row per lane is conflict-free)
constexpr int T5_OFF_QSTAGE = T5_SLOTS * T5_TILE;
constexpr int T5_OFF_BAR = T5_OFF_QSTAGE + T5_Q * T5_QPITCH * 4;
constexpr int T5_SMEM = T5_OFF_BAR + 256;
static_assert(T5_SMEM <= 227 * 1024, "shared memory budget");
static_assert(T5_Q * 2 * (T5_HD + 2) * 4 <= T5_SLOTS * T5_TILE, "the records are staged in the ring");
constexpr int T5_THREADS = 192;
// tensor memory: two score buffers of 128 columns (P overlays the first 64 of its buffer), the output, the query operand
constexpr uint32_t T5_TM_S = 0, T5_TM_O = 256, T5_TM_Q = 384, T5_TM_COLS = 512;
constexpr float T5_RESCALE = 8.0f;   // log2 units: rescale when the maximum grows by more than this (P stays below 2^8)

__device__ __forceinline__ float ex2f(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_h2f(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ void split_pair_f(float a, float b, uint32_t& hi, uint32_t& lo) {
    const __half2 h = __floats2half2_rn(a, b);
    const float2 back = __half22float2(h);
    const __half2 l = __floats2half2_rn(a - back.x, b - back.y);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = *reinterpret_cast<const uint32_t*>(&l);
}
}  // namespace

__global__ void __launch_bounds__(T5_THREADS, 1)
attn_t5_kernel(AttnGeom g, const float* q_rot, const __half* k_cache, const __half* v_cache, uint32_t start, int n_rows, float* partials,
               int chunks_per_span, float rescale_above, int* err) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ring = smem;
    float* q_stage = reinterpret_cast<float*>(smem + T5_OFF_QSTAGE);   // [64][129] f32: the queries, loaded row by row
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + T5_OFF_BAR);   // [6] a slot's tile has landed
    uint64_t* empty = full + T5_SLOTS;        // [6] the MMAs that read the slot have completed
    uint64_t* s_ready = empty + T5_SLOTS;     // [2] S = Q K^T of a tile is in tensor memory
    uint64_t* p_ready = s_ready + 2;          // [2] P (and a rescaled O) are in tensor memory
    uint64_t* pv_done = p_ready + 2;          // [2] O += P V of a tile has completed: its score buffer is free, O is at rest
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
    const int span = blockIdx.x, kvh = blockIdx.y;
    const uint32_t n_pos = start + (uint32_t)n_rows;
    const int c_begin = span * chunks_per_span;
    int c_end = (int)((n_pos + KV_TILE_KEYS - 1) / KV_TILE_KEYS);
    if (c_end > c_begin + chunks_per_span) c_end = c_begin + chunks_per_span;
    const int n_c = c_end - c_begin;   // >= 1 by the launch geometry

    if (threadIdx.x == 0) {
        for (int i = 0; i < T5_SLOTS; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&s_ready[i], 1);
            mbar_init(&p_ready[i], 4);
            mbar_init(&pv_done[i], 1);
        }
        abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 4) tmem_alloc(&tmem_slot, T5_TM_COLS);
    pdl_launch_dependents();
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem = tmem_slot;

    if (warp < 4) {
        // ================= softmax / rescale / epilogue: thread = tensor-memory lane =================
        const int L = 32 * warp + lane, q = L & 63, half = L >> 6, tok = q >> 2;
        const uint32_t tm_lane = tmem + ((uint32_t)(32 * warp) << 16);
        pdl_wait();   // the rotated queries come from the kernel before
        {
            // the 64 queries (pair = row * 4 + head-in-group) into shared memory with coalesced loads, then each lane takes
            // its own: scaled by log2(e) / sqrt(hd) (scores live in the exp2 domain) and split into an exact f16 hi + lo
            // pair; columns 0-63 of the operand = hi plane (k = 0..127), 64-127 = lo plane
            for (int idx = L; idx < T5_Q * (T5_HD / 4); idx += 128) {
                const int pair = idx / (T5_HD / 4), d4 = (idx % (T5_HD / 4)) * 4;
                const int row = pair / T5_GROUP;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (row < n_rows) v = *reinterpret_cast<const float4*>(q_rot + ((uint64_t)row * g.n_q + kvh * T5_GROUP + pair % T5_GROUP) * T5_HD + d4);
                float* dst = q_stage + pair * T5_QPITCH + d4;
                dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");   // the four softmax warps
            const float scale = 1.4426950408889634f / sqrtf((float)T5_HD);
            const float* src = q_stage + q * T5_QPITCH;
#pragma unroll
            for (int c = 0; c < 2; ++c) {   // 64 dims at a time
                uint32_t hi[32], lo[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) split_pair_f(src[64 * c + 2 * j] * scale, src[64 * c + 2 * j + 1] * scale, hi[j], lo[j]);
                tmem_st32(tm_lane + T5_TM_Q + 32 * c, hi);
                tmem_st32(tm_lane + T5_TM_Q + 64 + 32 * c, lo);
            }
            wait_st();
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_ready[1]);   // phase 0 of p_ready[1] doubles as "the query operand is written"
        }
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
        for (int i = 0; i < n_c && ok; ++i) {
            const int b = i & 1;
            if (__any_sync(0xffffffffu, *reinterpret_cast<volatile int*>(&abort_flag) != 0)) { ok = false; break; }
            ok = mbar_wait_spin(&s_ready[b], (uint32_t)(i >> 1) & 1u, err, DEV_ERR_WAIT_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            fence_after_sync();
            float s[64];
            {
                float t0[32], t1[32];
                tmem_ld32(tm_lane + T5_TM_S + 128 * b + 64 * half, t0);
                tmem_ld32(tm_lane + T5_TM_S + 128 * b + 64 * half + 32, t1);
                wait_ld();
#pragma unroll
                for (int j = 0; j < 32; ++j) { s[j] = t0[j]; s[32 + j] = t1[j]; }
            }
            const uint32_t p0 = (uint32_t)(c_begin + i) * KV_TILE_KEYS + 64u * (uint32_t)half;   // position of this lane's first key
            if (p0 + 64u > start + 1u) {
                // keys visible to the query: positions <= start + tok; rows beyond the call see nothing
                const long long lim = tok < n_rows ? (long long)start + tok + 1 - (long long)p0 : 0;
#pragma unroll
                for (int j = 0; j < 64; ++j)
                    if ((long long)j >= lim) s[j] = -INFINITY;
            }
            float mx[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) mx[j] = s[j];
#pragma unroll
            for (int j = 8; j < 64; ++j) mx[j & 7] = fmaxf(mx[j & 7], s[j]);
            const float mc = fmaxf(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])), fmaxf(fmaxf(mx[4], mx[5]), fmaxf(mx[6], mx[7])));
            const bool need = mc > m_ref + rescale_above;   // also the first finite maximum (m_ref = -inf)
            if (__any_sync(0xffffffffu, need)) {
                const float alpha = need ? ex2f(m_ref - mc) : 1.0f;   // 0 when there was no maximum yet
                if (i >= 1) {
                    // O must be at rest: the previous tile's O += P V has completed
                    ok = mbar_wait_spin(&pv_done[(i - 1) & 1], (uint32_t)((i - 1) >> 1) & 1u, err, DEV_ERR_WAIT_EMPTY);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    fence_after_sync();
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        float o[32];
                        tmem_ld32(tm_lane + T5_TM_O + 32 * c, o);
                        wait_ld();
                        uint32_t r[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(o[j] * alpha);
                        tmem_st32(tm_lane + T5_TM_O + 32 * c, r);
                    }
                }
                l *= alpha;
                if (need) m_ref = mc;
            }
            const float ms = m_ref > -INFINITY ? m_ref : 0.f;   // exp2(-inf - ms) = 0, never NaN
            float sum[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t pr[32], zero[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const float e0 = ex2f(s[2 * j] - ms), e1 = ex2f(s[2 * j + 1] - ms);
                sum[j & 3] += e0 + e1;
                pr[j] = pack_h2f(e0, e1);
                zero[j] = 0u;
            }
            l += (sum[0] + sum[1]) + (sum[2] + sum[3]);
            // P over the scores it came from: this lane's keys in its half of the 64 columns, zeros in the other half
            tmem_st32(tm_lane + T5_TM_S + 128 * b + 32 * half, pr);
            tmem_st32(tm_lane + T5_TM_S + 128 * b + 32 * (half ^ 1), zero);
            wait_st();
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_ready[b]);
        }
        if (ok) {
            ok = mbar_wait_spin(&pv_done[(n_c - 1) & 1], (uint32_t)((n_c - 1) >> 1) & 1u, err, DEV_ERR_WAIT_EMPTY);
            ok = __all_sync(0xffffffffu, ok);
        }
        if (!ok) abort_flag = 1;
        fence_after_sync();
        // one record per (span, key half, kv head, query): [m, l, O[128]], m back in the natural-log domain.  The two
        // groups of 64 records are contiguous in global memory; they are laid out in the ring (idle by now: every tile
        // has been consumed) and written with coalesced stores.
        float* stage = reinterpret_cast<float*>(ring) + (uint64_t)L * (T5_HD + 2);
        stage[0] = ok ? m_ref * 0.6931471805599453f : -INFINITY;
        stage[1] = ok ? l : 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            float o[32];
            tmem_ld32(tm_lane + T5_TM_O + 32 * c, o);
            wait_ld();
#pragma unroll
            for (int j = 0; j < 32; j += 2) *reinterpret_cast<float2*>(stage + 2 + 32 * c + j) = make_float2(o[j], o[j + 1]);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        constexpr int REC2 = T5_Q * (T5_HD + 2) / 2;   // float2 per group of 64 records
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            float2* dst = reinterpret_cast<float2*>(partials + ((uint64_t)(2 * span + hh) * g.n_kv + kvh) * T5_Q * (T5_HD + 2));
            const float2* src2 = reinterpret_cast<const float2*>(ring) + hh * REC2;
            for (int idx = L; idx < REC2; idx += 128) dst[idx] = src2[idx];
        }
    } else if (warp == 4) {
        // ================= MMA issue =================
        constexpr uint32_t IDESC = instr_desc(128);
        const uint32_t ring_addr = smem_u32(ring);
        // the query operand: p_ready[1] counts the four softmax warps once before its first use for a tile (tile 1 waits
        // for its phase 1)
        bool ok = mbar_wait_spin(&p_ready[1], 0u, err, DEV_ERR_WAIT_FULL);
        ok = __all_sync(0xffffffffu, ok);
        auto issue_qk = [&](int i) {
            const int b = i & 1, slot = (2 * i) % T5_SLOTS;
            ok = mbar_wait_spin(&full[slot], (uint32_t)((2 * i) / T5_SLOTS) & 1u, err, DEV_ERR_WAIT_FULL);
            // the buffer's P was the operand of the tile two steps back
            if (ok && i >= 2) ok = mbar_wait_spin(&pv_done[b], (uint32_t)((i >> 1) - 1) & 1u, err, DEV_ERR_WAIT_EMPTY);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) return;
            fence_after_sync();
            if (elect_one()) {
                const uint32_t k_addr = ring_addr + (uint32_t)slot * T5_TILE;
#pragma unroll
                for (int j = 0; j < 16; ++j)   // k steps of 16: the hi plane against the tile, then the lo plane against it again
                    mma_ts_rt(tmem + T5_TM_S + 128u * (uint32_t)b, tmem + T5_TM_Q + 8u * (uint32_t)j,
                              smem_desc(k_addr + (uint32_t)(j & 7) * 4096u, 2048, 128), IDESC, j > 0 ? 1u : 0u);
                mma_commit(&s_ready[b]);
                mma_commit(&empty[slot]);
            }
            __syncwarp();
        };
        if (ok) issue_qk(0);
        for (int i = 0; i < n_c && ok; ++i) {
            if (__any_sync(0xffffffffu, *reinterpret_cast<volatile int*>(&abort_flag) != 0)) { ok = false; break; }
            if (i + 1 < n_c) {
                issue_qk(i + 1);
                if (!ok) break;
            }
            const int b = i & 1, slot = (2 * i + 1) % T5_SLOTS;
            // tile 1's P arrives in phase 1 of p_ready[1] (phase 0 announced the query operand)
            const uint32_t p_phase = b == 1 ? (uint32_t)((i >> 1) + 1) & 1u : (uint32_t)(i >> 1) & 1u;
            ok = mbar_wait_spin(&p_ready[b], p_phase, err, DEV_ERR_WAIT_FULL);
            if (ok) ok = mbar_wait_spin(&full[slot], (uint32_t)((2 * i + 1) / T5_SLOTS) & 1u, err, DEV_ERR_WAIT_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            fence_after_sync();
            if (elect_one()) {
                const uint32_t v_addr = ring_addr + (uint32_t)slot * T5_TILE;
#pragma unroll
                for (int j = 0; j < 8; ++j)   // 16 keys per step
                    mma_ts_rt(tmem + T5_TM_O, tmem + T5_TM_S + 128u * (uint32_t)b + 8u * (uint32_t)j, smem_desc(v_addr + (uint32_t)j * 4096u, 2048, 128),
                              IDESC, (i > 0 || j > 0) ? 1u : 0u);
                mma_commit(&empty[slot]);
                mma_commit(&pv_done[b]);
            }
            __syncwarp();
        }
        if (!ok) abort_flag = 1;
    } else {
        // ================= producer =================
        if (lane == 0) {
            pdl_wait();   // the block's own K / V rows come from the kernel before
            bool ok = true;
            int issued = 0;
            const int n_t = 2 * n_c;   // tiles: K of tile i, V of tile i, K of tile i + 1, ...
            for (int t = 0; t < n_t && ok; ++t) {
                const int slot = t % T5_SLOTS;
                if (*reinterpret_cast<volatile int*>(&abort_flag)) break;
                if (t >= T5_SLOTS) ok = mbar_wait_bounded(&empty[slot], (uint32_t)(t / T5_SLOTS - 1) & 1u, err, DEV_ERR_WAIT_EMPTY);
                if (!ok) break;
                const uint64_t tile = ((uint64_t)(c_begin + (t >> 1)) * g.n_kv + kvh) * (uint64_t)(KV_TILE_KEYS * T5_HD);
                mbar_arrive_expect_tx(&full[slot], T5_TILE);
                bulk_g2s(ring + slot * T5_TILE, ((t & 1) ? v_cache : k_cache) + tile, T5_TILE, &full[slot]);
                issued = t + 1;
            }
            if (!ok) abort_flag = 1;
            // nothing may still be in flight into this CTA's shared memory when it leaves
            for (int t = issued > T5_SLOTS ? issued - T5_SLOTS : 0; t < issued; ++t)
                mbar_wait_bounded(&full[t % T5_SLOTS], (uint32_t)(t / T5_SLOTS) & 1u, err, DEV_ERR_WAIT_DRAIN);
        }
    }
    fence_before_sync();
    __syncthreads();
    if (warp == 4) {
        fence_after_sync();
        tmem_free(tmem, T5_TM_COLS);
    }
}

// ---- the drafter's attention on the same scheme ---------------------------------------------------------------------
// Queries = the block's noise rows; keys = the context columns followed by the noise rows' own K / V;
// allowed(q, k) = !causal || k_pos <= q_pos (kernels/dflash_attn.metal:99-103; sliding-window layers keep the mma.sync
// kernel, their span is short).  The drafter's context cache holds f32 rows; layers that attend over the whole context
// of a long session keep a shadow of it as tiles - per (128 columns, KV head) four 32 KiB tiles: K hi, K lo, V hi, V lo,
// the exact f16 hi + lo split of the f32 values in the operand layouts of attn_t5_kernel - written when columns are
// appended (dctx_tile_kernel).  The noise rows are one more tile set, rebuilt per pass.  Per tile of 128 keys:
//   S = Qh Kh + Ql Kh + Qh Kl   (24 MMAs),   O += P Vh + P Vl   (16 MMAs),   P rounded to f16 as in the verify kernel,
// so the result keeps f32-class accuracy against the f32 cache, like the mma.sync kernel it replaces.  The key
// positions of a context tile are staged beside it (512 bytes) for the causal mask.  Six ring slots hold the four
// tiles of a step plus half of the next.
constexpr int D5_OFF_POS = T5_OFF_BAR + 256;           // [2][128] u32 key positions
constexpr int D5_SMEM = D5_OFF_POS + 2 * 128 * 4;
static_assert(D5_SMEM <= 227 * 1024, "shared memory budget");

__global__ void __launch_bounds__(T5_THREADS, 1)
dattn_t5_kernel(AttnGeom g, const float* q_rot, const __half* ctx_tiles, const __half* noise_tiles, const uint32_t* pos_ctx, int n_ctx,
                uint32_t noise_start, int n_rows, int causal, float* partials, int chunks_per_span, float rescale_above, int* err) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ring = smem;
    float* q_stage = reinterpret_cast<float*>(smem + T5_OFF_QSTAGE);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + T5_OFF_BAR);
    uint64_t* empty = full + T5_SLOTS;
    uint64_t* s_ready = empty + T5_SLOTS;
    uint64_t* p_ready = s_ready + 2;
    uint64_t* pv_done = p_ready + 2;
    uint32_t* kpos = reinterpret_cast<uint32_t*>(smem + D5_OFF_POS);
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
    const int span = blockIdx.x, kvh = blockIdx.y;
    const int n_ctx_chunks = (n_ctx + KV_TILE_KEYS - 1) / KV_TILE_KEYS;   // the noise rows are chunk n_ctx_chunks
    const int c_begin = span * chunks_per_span;
    int c_end = n_ctx_chunks + 1;
    if (c_end > c_begin + chunks_per_span) c_end = c_begin + chunks_per_span;
    const int n_c = c_end - c_begin;   // >= 1 by the launch geometry

    if (threadIdx.x == 0) {
        for (int i = 0; i < T5_SLOTS; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&s_ready[i], 1);
            mbar_init(&p_ready[i], 4);
            mbar_init(&pv_done[i], 1);
        }
        abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 4) tmem_alloc(&tmem_slot, T5_TM_COLS);
    pdl_launch_dependents();
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem = tmem_slot;

    if (warp < 4) {
        const int L = 32 * warp + lane, q = L & 63, half = L >> 6, tok = q >> 2;
        const uint32_t tm_lane = tmem + ((uint32_t)(32 * warp) << 16);
        pdl_wait();
        {
            for (int idx = L; idx < T5_Q * (T5_HD / 4); idx += 128) {
                const int pair = idx / (T5_HD / 4), d4 = (idx % (T5_HD / 4)) * 4;
                const int row = pair / T5_GROUP;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (row < n_rows) v = *reinterpret_cast<const float4*>(q_rot + ((uint64_t)row * g.n_q + kvh * T5_GROUP + pair % T5_GROUP) * T5_HD + d4);
                float* dst = q_stage + pair * T5_QPITCH + d4;
                dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            const float scale = 1.4426950408889634f / sqrtf((float)T5_HD);
            const float* src = q_stage + q * T5_QPITCH;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t hi[32], lo[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) split_pair_f(src[64 * c + 2 * j] * scale, src[64 * c + 2 * j + 1] * scale, hi[j], lo[j]);
                tmem_st32(tm_lane + T5_TM_Q + 32 * c, hi);
                tmem_st32(tm_lane + T5_TM_Q + 64 + 32 * c, lo);
            }
            wait_st();
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_ready[1]);   // phase 0 of p_ready[1]: the query operand is written
        }
        const uint32_t q_pos = noise_start + (uint32_t)tok;
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
        for (int i = 0; i < n_c && ok; ++i) {
            const int b = i & 1, chunk = c_begin + i;
            if (__any_sync(0xffffffffu, *reinterpret_cast<volatile int*>(&abort_flag) != 0)) { ok = false; break; }
            ok = mbar_wait_spin(&s_ready[b], (uint32_t)(i >> 1) & 1u, err, DEV_ERR_WAIT_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            fence_after_sync();
            float s[64];
            {
                float t0[32], t1[32];
                tmem_ld32(tm_lane + T5_TM_S + 128 * b + 64 * half, t0);
                tmem_ld32(tm_lane + T5_TM_S + 128 * b + 64 * half + 32, t1);
                wait_ld();
#pragma unroll
                for (int j = 0; j < 32; ++j) { s[j] = t0[j]; s[32 + j] = t1[j]; }
            }
            const bool noise = chunk == n_ctx_chunks;
            const int k0 = 64 * half;   // this lane's first key inside the tile
            if (tok >= n_rows) {
#pragma unroll
                for (int j = 0; j < 64; ++j) s[j] = -INFINITY;
            } else if (noise) {
                // keys = the block's own rows: row j is visible when it exists and (bidirectional, or not after the query)
#pragma unroll
                for (int j = 0; j < 64; ++j) {
                    const int kj = k0 + j;
                    if (kj >= n_rows || (causal && kj > tok)) s[j] = -INFINITY;
                }
            } else if (causal || (chunk + 1) * KV_TILE_KEYS > n_ctx) {
                // positions were staged with the tile's first plane: observe that copy's barrier before reading them (the
                // phase completed long ago; the slot's next use cannot complete before this step's P is written)
                if (causal) {
                    const int u0 = 4 * i;
                    ok = mbar_wait_spin(&full[u0 % T5_SLOTS], (uint32_t)(u0 / T5_SLOTS) & 1u, err, DEV_ERR_WAIT_FULL);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                }
                const uint32_t* kp = kpos + 128 * b + k0;
                const int lim = n_ctx - chunk * KV_TILE_KEYS - k0;   // columns of this half that exist
#pragma unroll
                for (int j = 0; j < 64; ++j)
                    if (j >= lim || (causal && kp[j] > q_pos)) s[j] = -INFINITY;
            }
            float mx[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) mx[j] = s[j];
#pragma unroll
            for (int j = 8; j < 64; ++j) mx[j & 7] = fmaxf(mx[j & 7], s[j]);
            const float mc = fmaxf(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])), fmaxf(fmaxf(mx[4], mx[5]), fmaxf(mx[6], mx[7])));
            const bool need = mc > m_ref + rescale_above;
            if (__any_sync(0xffffffffu, need)) {
                const float alpha = need ? ex2f(m_ref - mc) : 1.0f;
                if (i >= 1) {
                    ok = mbar_wait_spin(&pv_done[(i - 1) & 1], (uint32_t)((i - 1) >> 1) & 1u, err, DEV_ERR_WAIT_EMPTY);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    fence_after_sync();
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        float o[32];
                        tmem_ld32(tm_lane + T5_TM_O + 32 * c, o);
                        wait_ld();
                        uint32_t r[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(o[j] * alpha);
                        tmem_st32(tm_lane + T5_TM_O + 32 * c, r);
                    }
                }
                l *= alpha;
                if (need) m_ref = mc;
            }
            const float ms = m_ref > -INFINITY ? m_ref : 0.f;
            float sum[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t pr[32], zero[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const float e0 = ex2f(s[2 * j] - ms), e1 = ex2f(s[2 * j + 1] - ms);
                sum[j & 3] += e0 + e1;
                pr[j] = pack_h2f(e0, e1);
                zero[j] = 0u;
            }
            l += (sum[0] + sum[1]) + (sum[2] + sum[3]);
            tmem_st32(tm_lane + T5_TM_S + 128 * b + 32 * half, pr);
            tmem_st32(tm_lane + T5_TM_S + 128 * b + 32 * (half ^ 1), zero);
            wait_st();
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_ready[b]);
        }
        if (ok) {
            ok = mbar_wait_spin(&pv_done[(n_c - 1) & 1], (uint32_t)((n_c - 1) >> 1) & 1u, err, DEV_ERR_WAIT_EMPTY);
            ok = __all_sync(0xffffffffu, ok);
        }
        if (!ok) abort_flag = 1;
        fence_after_sync();
        float* stage = reinterpret_cast<float*>(ring) + (uint64_t)L * (T5_HD + 2);
        stage[0] = ok ? m_ref * 0.6931471805599453f : -INFINITY;
        stage[1] = ok ? l : 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            float o[32];
            tmem_ld32(tm_lane + T5_TM_O + 32 * c, o);
            wait_ld();
#pragma unroll
            for (int j = 0; j < 32; j += 2) *reinterpret_cast<float2*>(stage + 2 + 32 * c + j) = make_float2(o[j], o[j + 1]);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        constexpr int REC2 = T5_Q * (T5_HD + 2) / 2;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            float2* dst = reinterpret_cast<float2*>(partials + ((uint64_t)(2 * span + hh) * g.n_kv + kvh) * T5_Q * (T5_HD + 2));
            const float2* src2 = reinterpret_cast<const float2*>(ring) + hh * REC2;
            for (int idx = L; idx < REC2; idx += 128) dst[idx] = src2[idx];
        }
    } else if (warp == 4) {
        constexpr uint32_t IDESC = instr_desc(128);
        const uint32_t ring_addr = smem_u32(ring);
        bool ok = mbar_wait_spin(&p_ready[1], 0u, err, DEV_ERR_WAIT_FULL);
        ok = __all_sync(0xffffffffu, ok);
        // tile u of this CTA (four per step: K hi, K lo, V hi, V lo) lives in ring slot u % 6, use u / 6
        auto wait_tile = [&](int u) { return mbar_wait_spin(&full[u % T5_SLOTS], (uint32_t)(u / T5_SLOTS) & 1u, err, DEV_ERR_WAIT_FULL); };
        auto issue_qk = [&](int i) {
            const int b = i & 1, u = 4 * i;
            ok = wait_tile(u) && wait_tile(u + 1);
            if (ok && i >= 2) ok = mbar_wait_spin(&pv_done[b], (uint32_t)((i >> 1) - 1) & 1u, err, DEV_ERR_WAIT_EMPTY);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) return;
            fence_after_sync();
            if (elect_one()) {
                const uint32_t kh = ring_addr + (uint32_t)(u % T5_SLOTS) * T5_TILE, kl = ring_addr + (uint32_t)((u + 1) % T5_SLOTS) * T5_TILE;
#pragma unroll
                for (int j = 0; j < 24; ++j) {   // Qh Kh, Ql Kh, Qh Kl: eight k steps of 16 dims each
                    const uint32_t a_col = j < 8 ? 8u * j : j < 16 ? 64u + 8u * (j - 8) : 8u * (j - 16);
                    const uint32_t k_addr = (j < 16 ? kh : kl) + (uint32_t)(j & 7) * 4096u;
                    mma_ts_rt(tmem + T5_TM_S + 128u * (uint32_t)b, tmem + T5_TM_Q + a_col, smem_desc(k_addr, 2048, 128), IDESC, j > 0 ? 1u : 0u);
                }
                mma_commit(&s_ready[b]);
                mma_commit(&empty[u % T5_SLOTS]);
                mma_commit(&empty[(u + 1) % T5_SLOTS]);
            }
            __syncwarp();
        };
        if (ok) issue_qk(0);
        for (int i = 0; i < n_c && ok; ++i) {
            if (__any_sync(0xffffffffu, *reinterpret_cast<volatile int*>(&abort_flag) != 0)) { ok = false; break; }
            if (i + 1 < n_c) {
                issue_qk(i + 1);
                if (!ok) break;
            }
            const int b = i & 1, u = 4 * i + 2;
            const uint32_t p_phase = b == 1 ? (uint32_t)((i >> 1) + 1) & 1u : (uint32_t)(i >> 1) & 1u;
            ok = mbar_wait_spin(&p_ready[b], p_phase, err, DEV_ERR_WAIT_FULL);
            if (ok) ok = wait_tile(u) && wait_tile(u + 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            fence_after_sync();
            if (elect_one()) {
                const uint32_t vh = ring_addr + (uint32_t)(u % T5_SLOTS) * T5_TILE, vl = ring_addr + (uint32_t)((u + 1) % T5_SLOTS) * T5_TILE;
#pragma unroll
                for (int j = 0; j < 16; ++j)   // P Vh, then P Vl: 16 keys per step
                    mma_ts_rt(tmem + T5_TM_O, tmem + T5_TM_S + 128u * (uint32_t)b + 8u * (uint32_t)(j & 7),
                              smem_desc((j < 8 ? vh : vl) + (uint32_t)(j & 7) * 4096u, 2048, 128), IDESC, (i > 0 || j > 0) ? 1u : 0u);
                mma_commit(&empty[u % T5_SLOTS]);
                mma_commit(&empty[(u + 1) % T5_SLOTS]);
                mma_commit(&pv_done[b]);
            }
            __syncwarp();
        }
        if (!ok) abort_flag = 1;
    } else {
        if (lane == 0) {
            pdl_wait();
            bool ok = true;
            int issued = 0;
            const int n_t = 4 * n_c;
            for (int t = 0; t < n_t && ok; ++t) {
                const int slot = t % T5_SLOTS, i = t >> 2, plane = t & 3, chunk = c_begin + i;
                if (*reinterpret_cast<volatile int*>(&abort_flag)) break;
                if (t >= T5_SLOTS) ok = mbar_wait_bounded(&empty[slot], (uint32_t)(t / T5_SLOTS - 1) & 1u, err, DEV_ERR_WAIT_EMPTY);
                if (!ok) break;
                const bool noise = chunk == n_ctx_chunks;
                const __half* src = noise ? noise_tiles + ((uint64_t)kvh * 4 + plane) * (uint64_t)(KV_TILE_KEYS * T5_HD)
                                          : ctx_tiles + (((uint64_t)chunk * g.n_kv + kvh) * 4 + plane) * (uint64_t)(KV_TILE_KEYS * T5_HD);
                // the key positions of a context tile ride on the barrier of its first plane (the buffer of step i - 2 was
                // last read by that step's softmax, which completed before the slot's previous tile was released)
                const bool with_pos = plane == 0 && !noise;
                mbar_arrive_expect_tx(&full[slot], T5_TILE + (with_pos ? 512u : 0u));
                bulk_g2s(ring + slot * T5_TILE, src, T5_TILE, &full[slot]);
                if (with_pos) bulk_g2s(kpos + 128 * (i & 1), pos_ctx + (uint64_t)chunk * KV_TILE_KEYS, 512, &full[slot]);
                issued = t + 1;
            }
            if (!ok) abort_flag = 1;
            for (int t = issued > T5_SLOTS ? issued - T5_SLOTS : 0; t < issued; ++t)
                mbar_wait_bounded(&full[t % T5_SLOTS], (uint32_t)(t / T5_SLOTS) & 1u, err, DEV_ERR_WAIT_DRAIN);
        }
    }
    fence_before_sync();
    __syncthreads();
    if (warp == 4) {
        fence_after_sync();
        tmem_free(tmem, T5_TM_COLS);
    }
}

// f32 K / V rows [first, first + count) of a position-major cache -> their f16 hi + lo tiles (row index = key index)
__global__ void dctx_tile_kernel(const float* k_rows, const float* v_rows, int n_kv, uint32_t first, uint32_t count, uint32_t row0, __half* tiles) {
    pdl_prologue();
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;   // one element of one row
    const uint64_t per_row = (uint64_t)n_kv * T5_HD;
    if (i >= (uint64_t)count * per_row) return;
    const uint32_t r = (uint32_t)(i / per_row);
    const int h = (int)((i % per_row) / T5_HD), d = (int)(i % T5_HD);
    const uint32_t key_index = first + r;                                   // position of the row in the tiled sequence
    const uint64_t src = ((uint64_t)(row0 + r) * n_kv + h) * T5_HD + d;
    __half* base = tiles + (((uint64_t)(key_index / KV_TILE_KEYS) * n_kv + h) * 4) * (uint64_t)(KV_TILE_KEYS * T5_HD);
    const uint32_t key = key_index % KV_TILE_KEYS;
    const float kf = k_rows[src], vf = v_rows[src];
    const __half khi = __float2half_rn(kf), vhi = __float2half_rn(vf);
    const uint32_t ko = kv_tile_k_off(key, d), vo = kv_tile_v_off(key, d);
    constexpr uint64_t PLANE = (uint64_t)KV_TILE_KEYS * T5_HD;
    base[ko] = khi;
    base[PLANE + ko] = __float2half_rn(kf - __half2float(khi));
    base[2 * PLANE + vo] = vhi;
    base[3 * PLANE + vo] = __float2half_rn(vf - __half2float(vhi));
}

uint64_t dattn_t5_tile_halfs(int n_kv, uint32_t n_keys) { return ((uint64_t)(n_keys + KV_TILE_KEYS - 1) / KV_TILE_KEYS) * n_kv * 4 * (uint64_t)(KV_TILE_KEYS * T5_HD); }

// rows [row0, row0 + count) of the f32 caches become keys [first, first + count) of the tiled sequence
dfl_status launch_dctx_tiles(cudaStream_t st, const float* k_rows, const float* v_rows, int n_kv, uint32_t first, uint32_t count, uint32_t row0,
                             void* tiles) {
    if (count == 0) return DFL_OK;
    const uint64_t n = (uint64_t)count * n_kv * T5_HD;
    launch_k(dctx_tile_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, k_rows, v_rows, n_kv, first, count, row0, reinterpret_cast<__half*>(tiles));
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

dfl_status launch_dattn_t5(cudaStream_t st, const AttnGeom& g, const float* q_rot, const void* ctx_tiles, const void* noise_tiles,
                           const uint32_t* pos_ctx, int n_ctx, uint32_t noise_start, int n_rows, bool causal, float* partials, uint32_t ctx_capacity,
                           int* err, int* n_records_out) {
    static std::once_flag once[16];
    int dev = 0;
    DFL_CUDA(cudaGetDevice(&dev));
    cudaError_t attr = cudaSuccess;
    std::call_once(once[dev & 15], [&] { attr = cudaFuncSetAttribute(dattn_t5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, D5_SMEM); });
    DFL_CUDA(attr);
    const int cps = attn_t5_chunks_per_span(g, ctx_capacity + KV_TILE_KEYS);
    const int n_chunks = (n_ctx + KV_TILE_KEYS - 1) / KV_TILE_KEYS + 1;
    const int n_spans = (n_chunks + cps - 1) / cps;
    float rescale_above = T5_RESCALE;
    if (const char* e = getenv("DFL_ATTN_T5_RESCALE")) {
        const float v = (float)atof(e);
        if (v >= 0.f && v <= 12.f) rescale_above = v;
    }
    launch_k(dattn_t5_kernel, dim3((unsigned)n_spans, (unsigned)g.n_kv), dim3(T5_THREADS), (size_t)D5_SMEM, st, g, q_rot,
              reinterpret_cast<const __half*>(ctx_tiles), reinterpret_cast<const __half*>(noise_tiles), pos_ctx, n_ctx, noise_start, n_rows,
              causal ? 1 : 0, partials, cps, rescale_above, err);
    count_launch();
    DFL_CUDA(cudaGetLastError());
    *n_records_out = 2 * n_spans;
    return DFL_OK;
}

bool attn_t5_supported(const AttnGeom& g, bool kv_f16) { return kv_f16 && g.hd == T5_HD && g.n_q / g.n_kv == T5_GROUP; }

// tiles per span from the session's KV capacity only (never from the call): one CTA per SM and one wave at full
// capacity - as many spans per KV head as whole heads' worth of CTAs fit on the SMs
int attn_t5_chunks_per_span(const AttnGeom& g, uint32_t kv_capacity) {
    const uint64_t cap_chunks = ((uint64_t)kv_capacity + KV_TILE_KEYS - 1) / KV_TILE_KEYS;
    uint64_t slots = (uint64_t)sm_count() / (uint64_t)g.n_kv * (uint64_t)g.n_kv;
    if (slots < (uint64_t)g.n_kv) slots = (uint64_t)g.n_kv;
    uint64_t b = (cap_chunks * g.n_kv + slots - 1) / slots;
    if (b < 1) b = 1;
    return (int)b;
}

dfl_status launch_attn_t5(cudaStream_t st, const AttnGeom& g, const float* q_rot, const void* k_cache, const void* v_cache, uint32_t start,
                          int n_rows, float* partials, int chunks_per_span, int* err) {
    static std::once_flag once[16];
    int dev = 0;
    DFL_CUDA(cudaGetDevice(&dev));
    cudaError_t attr = cudaSuccess;
    std::call_once(once[dev & 15], [&] { attr = cudaFuncSetAttribute(attn_t5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T5_SMEM); });
    DFL_CUDA(attr);
    const int n_chunks = (int)((start + (uint32_t)n_rows + KV_TILE_KEYS - 1) / KV_TILE_KEYS);
    const int n_spans = (n_chunks + chunks_per_span - 1) / chunks_per_span;
    // DFL_ATTN_T5_RESCALE (test hook): the growth of a lane's maximum, in log2 units within [0, 12], above which the
    // output is rescaled; 0 rescales at every new maximum.  Results must agree with the oracle at any setting.
    float rescale_above = T5_RESCALE;
    if (const char* e = getenv("DFL_ATTN_T5_RESCALE")) {
        const float v = (float)atof(e);
        if (v >= 0.f && v <= 12.f) rescale_above = v;
    }
    launch_k(attn_t5_kernel, dim3((unsigned)n_spans, (unsigned)g.n_kv), dim3(T5_THREADS), (size_t)T5_SMEM, st, g, q_rot,
              reinterpret_cast<const __half*>(k_cache), reinterpret_cast<const __half*>(v_cache), start, n_rows, partials, chunks_per_span, rescale_above, err);
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

// ---- conversions between the tiled cache and position-major rows [pos][n_kv][128] (snapshots, host reads) ----
__global__ void kv_tiled_to_rows_kernel(const __half* tiled, int is_v, int n_kv, uint32_t pos0, uint32_t n_pos, __half* rows) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;   // one element
    const uint64_t per_pos = (uint64_t)n_kv * T5_HD;
    if (i >= (uint64_t)n_pos * per_pos) return;
    const uint32_t pos = pos0 + (uint32_t)(i / per_pos);
    const int h = (int)((i % per_pos) / T5_HD), d = (int)(i % T5_HD);
    const uint64_t src = kv_tile_base(pos, n_kv, h) + (is_v ? kv_tile_v_off(pos & (KV_TILE_KEYS - 1), d) : kv_tile_k_off(pos & (KV_TILE_KEYS - 1), d));
    rows[i] = tiled[src];
}
__global__ void kv_rows_to_tiled_kernel(const __half* rows, int is_v, int n_kv, uint32_t pos0, uint32_t n_pos, __half* tiled) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t per_pos = (uint64_t)n_kv * T5_HD;
    if (i >= (uint64_t)n_pos * per_pos) return;
    const uint32_t pos = pos0 + (uint32_t)(i / per_pos);
    const int h = (int)((i % per_pos) / T5_HD), d = (int)(i % T5_HD);
    const uint64_t dst = kv_tile_base(pos, n_kv, h) + (is_v ? kv_tile_v_off(pos & (KV_TILE_KEYS - 1), d) : kv_tile_k_off(pos & (KV_TILE_KEYS - 1), d));
    tiled[dst] = rows[i];
}
dfl_status launch_kv_tiled_to_rows(cudaStream_t st, const void* tiled, bool is_v, int n_kv, uint32_t pos0, uint32_t n_pos, void* rows) {
    if (n_pos == 0) return DFL_OK;
    const uint64_t n = (uint64_t)n_pos * n_kv * T5_HD;
    kv_tiled_to_rows_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(reinterpret_cast<const __half*>(tiled), is_v ? 1 : 0, n_kv, pos0, n_pos,
                                                                        reinterpret_cast<__half*>(rows));
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}
dfl_status launch_kv_rows_to_tiled(cudaStream_t st, const void* rows, bool is_v, int n_kv, uint32_t pos0, uint32_t n_pos, void* tiled) {
    if (n_pos == 0) return DFL_OK;
    const uint64_t n = (uint64_t)n_pos * n_kv * T5_HD;
    kv_rows_to_tiled_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(reinterpret_cast<const __half*>(rows), is_v ? 1 : 0, n_kv, pos0, n_pos,
                                                                        reinterpret_cast<__half*>(tiled));
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

}  // namespace dfl
