// DFlash block-diffusion drafter: resident head, per-request drafter session and one draft
// pass (reference: MetalDFlashHead::load / MetalDFlashSession / draft_block_inner,
// crates/qwen-llm/src/metal_dflash.rs:4944-5050, :5492-5816, :15952-17164; oracle
// Forward::dflash_draft, crates/qwen-llm/src/forward.rs:380-662; attention mask
// kernels/dflash_attn.metal:99-103).
//
// The context side is incremental, as in the reference (watermark ctx_h_ready_n / kv_ctx_ready_n,
// metal_dflash.rs:16045-16143): fc + hidden_norm and every layer's K/V projection, K-norm and
// RoPE run once per appended context column and are kept in per-layer caches; a draft call only
// projects what was appended since the last call.
#include <algorithm>
#include <cstring>

#include "model.cuh"

namespace dfl {

struct DLayerW {
    float *attn_norm_w = nullptr, *post_norm_w = nullptr, *q_norm_w = nullptr, *k_norm_w = nullptr;
    MatGroup qkv, kv, wo, gate_up, down;
    bool is_swa = false;
};

// ---- drafter attention: queries = noise rows, keys = context cache || noise rows -----------
// allowed(q_pos, k_pos) = (!causal || k_pos <= q_pos) && (!swa || window == 0 || |q - k| < window)
template <int HD>
__global__ void __launch_bounds__(256) dattn_chunk_kernel(AttnGeom g, const float* q_rot, const float* k_ctx,
                                                          const float* v_ctx, const uint32_t* pos_ctx, int ctx_begin,
                                                          int n_ctx, const float* k_noise, const float* v_noise,
                                                          uint32_t noise_start, int n_rows, int causal, uint32_t window,
                                                          float* partials) {
    pdl_prologue();
    extern __shared__ float sm[];
    constexpr int LD = HD + 1;
    float* ks = sm;
    float* vs = ks + ATTN_CHUNK * LD;
    float* qs = vs + ATTN_CHUNK * LD;
    float* ps = qs + 8 * HD;
    __shared__ uint32_t kpos[ATTN_CHUNK];
    const int chunk = blockIdx.x, kvh = blockIdx.y;
    const int group = g.n_q / g.n_kv;
    const int n_keys = n_ctx + n_rows;
    const int j0 = chunk * ATTN_CHUNK;
    const int n_here = min(ATTN_CHUNK, n_keys - j0);
    for (int idx = threadIdx.x; idx < ATTN_CHUNK * HD; idx += blockDim.x) {
        const int kp = idx / HD, d = idx % HD;
        float kv = 0.f, vv = 0.f;
        if (kp < n_here) {
            const int j = j0 + kp;
            if (j < n_ctx) {
                const uint64_t o = ((uint64_t)(ctx_begin + j) * g.n_kv + kvh) * HD + d;
                kv = k_ctx[o];
                vv = v_ctx[o];
            } else {
                const uint64_t o = ((uint64_t)(j - n_ctx) * g.n_kv + kvh) * HD + d;
                kv = k_noise[o];
                vv = v_noise[o];
            }
        }
        ks[kp * LD + d] = kv;
        vs[kp * LD + d] = vv;
    }
    if (threadIdx.x < ATTN_CHUNK) {
        const int j = j0 + threadIdx.x;
        kpos[threadIdx.x] = j < n_ctx ? pos_ctx[ctx_begin + j] : noise_start + (uint32_t)(j - n_ctx);
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float scale = 1.0f / sqrtf((float)HD);
    const int n_queries = n_rows * group;
    float* myq = qs + warp * HD;
    float* myp = ps + warp * ATTN_CHUNK;
    for (int qi = warp; qi < n_queries; qi += 8) {
        const int row = qi / group, qh = kvh * group + qi % group;
        const float* qsrc = q_rot + ((uint64_t)row * g.n_q + qh) * HD;
        for (int d = lane; d < HD; d += 32) myq[d] = qsrc[d];
        __syncwarp();
        const uint32_t q_pos = noise_start + (uint32_t)row;
        float s0 = 0.f, s1 = 0.f;
        const float* k0 = ks + lane * LD;
        const float* k1 = ks + (lane + 32) * LD;
#pragma unroll 8
        for (int d = 0; d < HD; ++d) {
            const float qv = myq[d];
            s0 = fmaf(qv, k0[d], s0);
            s1 = fmaf(qv, k1[d], s1);
        }
        s0 *= scale;
        s1 *= scale;
        auto allowed = [&](int kp) {
            if (kp >= n_here) return false;
            const uint32_t kpv = kpos[kp];
            const uint32_t diff = q_pos > kpv ? q_pos - kpv : kpv - q_pos;
            return (!causal || kpv <= q_pos) && (window == 0 || diff < window);
        };
        const bool ok0 = allowed(lane), ok1 = allowed(lane + 32);
        if (!ok0) s0 = -INFINITY;
        if (!ok1) s1 = -INFINITY;
        const float m = warp_max(fmaxf(s0, s1));
        float e0 = 0.f, e1 = 0.f;
        if (m > -INFINITY) {
            e0 = ok0 ? expf(s0 - m) : 0.f;
            e1 = ok1 ? expf(s1 - m) : 0.f;
        }
        const float l = warp_sum(e0 + e1);
        myp[lane] = e0;
        myp[lane + 32] = e1;
        __syncwarp();
        float acc[HD / 32];
#pragma unroll
        for (int j = 0; j < HD / 32; ++j) acc[j] = 0.f;
        for (int kp = 0; kp < n_here; ++kp) {
            const float pw = myp[kp];
#pragma unroll
            for (int j = 0; j < HD / 32; ++j) acc[j] = fmaf(pw, vs[kp * LD + lane + 32 * j], acc[j]);
        }
        float* rec = partials + (((uint64_t)chunk * g.n_kv + kvh) * (MAX_ROWS * group) + qi) * (HD + 2);
        if (lane == 0) { rec[0] = m; rec[1] = l; }
#pragma unroll
        for (int j = 0; j < HD / 32; ++j) rec[2 + lane + 32 * j] = acc[j];
        __syncwarp();
    }
}

// combine over a fixed number of chunks + activation packing (rows >= n_rows packed as zeros)
template <int HD>
__global__ void __launch_bounds__(32) dattn_post_kernel(AttnGeom g, const float* partials, int n_chunks, int n_rows, uint8_t* acts,
                                                        int bf3, int* err) {
    pdl_prologue();
    constexpr int PER = HD / 32;
    const int qh = blockIdx.x, row = blockIdx.y, lane = threadIdx.x;
    const int group = g.n_q / g.n_kv, kvh = qh / group, qi = row * group + qh % group;
    float v[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) v[j] = 0.f;
    if (row < n_rows) {
        float M = -INFINITY;
        for (int c = lane; c < n_chunks; c += 32)
            M = fmaxf(M, partials[(((uint64_t)c * g.n_kv + kvh) * (MAX_ROWS * group) + qi) * (HD + 2)]);
        M = warp_max(M);
        float L = 0.f;
        // records merged in index order, their loads issued eight records at a time
        constexpr int BATCH = 8;
        const uint64_t rec_stride = (uint64_t)g.n_kv * (MAX_ROWS * group) * (HD + 2);
        const float* rec0 = partials + ((uint64_t)kvh * (MAX_ROWS * group) + qi) * (HD + 2);
        for (int c0 = 0; c0 < n_chunks; c0 += BATCH) {
            float mb[BATCH], lb[BATCH], vb[BATCH][PER];
#pragma unroll
            for (int u = 0; u < BATCH; ++u) {
                const float* rec = rec0 + (uint64_t)(c0 + u < n_chunks ? c0 + u : n_chunks - 1) * rec_stride;
                mb[u] = rec[0];
                lb[u] = rec[1];
#pragma unroll
                for (int j = 0; j < PER; ++j) vb[u][j] = rec[2 + lane * PER + j];
            }
#pragma unroll
            for (int u = 0; u < BATCH; ++u) {
                if (c0 + u >= n_chunks || mb[u] == -INFINITY) continue;
                const float f = expf(mb[u] - M);
                L = fmaf(lb[u], f, L);
#pragma unroll
                for (int j = 0; j < PER; ++j) v[j] = fmaf(vb[u][j], f, v[j]);
            }
        }
        const float inv = 1.0f / L;
#pragma unroll
        for (int j = 0; j < PER; ++j) v[j] *= inv;
    }
    const int col0 = qh * HD + lane * PER;
    bool over = false;
    float sum = 0.f;
#pragma unroll
    for (int q4 = 0; q4 < PER / 4; ++q4) {
        const int col = col0 + 4 * q4;
        uint8_t* chunk = acts + (uint64_t)(col >> 8) * act_chunk_dev(bf3);
        const float quad[4] = {v[4 * q4], v[4 * q4 + 1], v[4 * q4 + 2], v[4 * q4 + 3]};
        pack_quad_any(chunk, bf3, row, col & 255, quad, over);
        sum += quad[0] + quad[1] + quad[2] + quad[3];
    }
    if ((bf3 == ACT_F16 || bf3 == ACT_TS)) {
        constexpr int LANES = 32 / PER;
#pragma unroll
        for (int o = LANES / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if ((lane % LANES) == 0)
            store_subsum(acts + (uint64_t)(col0 >> 8) * act_chunk_dev(bf3), bf3, row, (col0 & 255) >> 5, sum, over);
    }
    if (over) atomicCAS(err, 0, DEV_ERR_OVERFLOW);
}

// merge of `n_records` records per query + packing (128-wide heads)
dfl_status launch_dattn_post(cudaStream_t st, const AttnGeom& g, const float* partials, int n_records, int n_rows, uint8_t* acts, int bf3, int* err) {
    launch_k(dattn_post_kernel<128>, dim3(dim3((unsigned)g.n_q, MAX_ROWS)), dim3(32), 0, st, g, partials, n_records, n_rows, acts, bf3, err);
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

dfl_status launch_drafter_attn(cudaStream_t st, const AttnGeom& g, const float* q_rot, const float* k_ctx, const float* v_ctx,
                               const int32_t* pos_ctx, int ctx_begin, int ctx_len, const float* k_noise, const float* v_noise,
                               uint32_t noise_start, int n_rows, bool causal, uint32_t window, float* partials, uint8_t* acts, int bf3,
                               int* err, uint32_t ctx_capacity) {
    const int n_ctx = ctx_len - ctx_begin;
    const int n_chunks = (n_ctx + n_rows + ATTN_CHUNK - 1) / ATTN_CHUNK;
    const uint32_t* pc = reinterpret_cast<const uint32_t*>(pos_ctx);
    // tensor-core span kernel for the usual geometry (DFL_DATTN_TC=0 keeps the scalar kernel)
    static const bool tc_enabled = [] { const char* e = getenv("DFL_DATTN_TC"); return !(e && e[0] == '0'); }();
    if (tc_enabled && ctx_capacity > 0 && dattn_tc_supported(g)) {
        int n_spans = 0;
        DFL_CHECK(launch_dattn_span_tc(st, g, q_rot, k_ctx, v_ctx, pc, ctx_begin, n_ctx, k_noise, v_noise, noise_start, n_rows, causal, window,
                                       partials, ctx_capacity, &n_spans));
        launch_k(dattn_post_kernel<128>, dim3(dim3((unsigned)g.n_q, MAX_ROWS)), dim3(32), 0, st, g, partials, n_spans, n_rows, acts, bf3, err);
        count_launch();
        DFL_CUDA(cudaGetLastError());
        return DFL_OK;
    }
    if (g.hd == 128) {
        const size_t smem = (size_t)(2 * ATTN_CHUNK * 129 + 8 * 128 + 8 * ATTN_CHUNK) * sizeof(float);
        static bool set = false;
        if (!set) { DFL_CUDA(cudaFuncSetAttribute(dattn_chunk_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); set = true; }
        launch_k(dattn_chunk_kernel<128>, dim3(dim3((unsigned)n_chunks, (unsigned)g.n_kv)), dim3(256), smem, st, g, q_rot, k_ctx, v_ctx, pc, ctx_begin, n_ctx, k_noise, v_noise,
                                                                                          noise_start, n_rows, causal ? 1 : 0, window, partials);
        launch_k(dattn_post_kernel<128>, dim3(dim3((unsigned)g.n_q, MAX_ROWS)), dim3(32), 0, st, g, partials, n_chunks, n_rows, acts, bf3, err);
    } else if (g.hd == 256) {
        const size_t smem = (size_t)(2 * ATTN_CHUNK * 257 + 8 * 256 + 8 * ATTN_CHUNK) * sizeof(float);
        static bool set = false;
        if (!set) { DFL_CUDA(cudaFuncSetAttribute(dattn_chunk_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); set = true; }
        launch_k(dattn_chunk_kernel<256>, dim3(dim3((unsigned)n_chunks, (unsigned)g.n_kv)), dim3(256), smem, st, g, q_rot, k_ctx, v_ctx, pc, ctx_begin, n_ctx, k_noise, v_noise,
                                                                                          noise_start, n_rows, causal ? 1 : 0, window, partials);
        launch_k(dattn_post_kernel<256>, dim3(dim3((unsigned)g.n_q, MAX_ROWS)), dim3(32), 0, st, g, partials, n_chunks, n_rows, acts, bf3, err);
    } else {
        return fail(DFL_ERR_UNSUPPORTED, "drafter attention: head_dim must be 128 or 256");
    }
    count_launch(2);
    DFL_CUDA(cudaGetLastError());
    return DFL_OK;
}

}  // namespace dfl

using namespace dfl;

struct dfl_drafter {
    const dfl_model* target = nullptr;
    dfl_dflash_config cfg{};
    MatGroup fc;
    float *hidden_norm_w = nullptr, *out_norm_w = nullptr;
    std::vector<DLayerW> layers;
    uint64_t weight_bytes = 0;
    // DFlash 2 path selector (metal_dflash.rs:2789-2797): the gate projection on the device, the codebooks on the host
    bool has_selector = false;
    MatGroup sel_hidden;
    dfl_codebook *sel_pred = nullptr, *sel_succ = nullptr;
    AttnGeom geom(int n_q) const {
        AttnGeom g;
        g.n_q = n_q; g.n_kv = (int)cfg.n_kv_heads; g.hd = (int)cfg.head_dim; g.n_rot = (int)cfg.head_dim;
        g.theta = cfg.rope_theta; g.eps = cfg.rms_norm_eps;
        return g;
    }
};

constexpr uint32_t kPendingCap = 256;  // appended-but-unprojected context columns kept in staging

struct dfl_dsession {
    const dfl_drafter* d = nullptr;
    uint32_t ctx_capacity = 0, ctx_len = 0, ready = 0;
    uint32_t pending_base = 0;          // column index of staging row 0
    float* staging = nullptr;           // [kPendingCap][K*H]
    uint32_t* pos_ctx_dev = nullptr;    // [capacity]
    std::vector<uint32_t> pos_host;
    std::vector<float*> k_ctx, v_ctx;   // per layer [capacity][n_kv][hd]
    // long sessions: per full-attention layer a shadow of the rows above as f16 hi + lo tiles for the tcgen05 attention
    // kernel (null for the other layers), and the tile set of the block's own rows
    std::vector<void*> ctx_tiles;
    void* noise_tiles = nullptr;
    // scratch
    float *x = nullptr, *part = nullptr, *sumsq = nullptr, *q_rot = nullptr, *k_noise = nullptr, *v_noise = nullptr, *attn_part = nullptr;
    uint8_t *acts_h = nullptr, *acts_f = nullptr, *acts_q = nullptr, *acts_fc = nullptr, *acts_lm = nullptr;
    float *logits = nullptr, *gap = nullptr;
    int32_t *argmax = nullptr, *tokens_dev = nullptr;
    void* am_scratch = nullptr;
    // top-16 per row and the selector's gate rows W_h h of the last pass
    int32_t* topk_ids = nullptr;
    float *topk_vals = nullptr, *sel_h = nullptr;
    void* topk_scratch = nullptr;
    uint8_t* acts_sel = nullptr;
    bool have_topk = false;
    uint8_t* pinned_sel = nullptr;   // [16][16] ids | [16][16] vals | [16][rank] gate rows
    // projection of newly appended context columns: its own scratch, so that it can run on a side stream beside the
    // start of the draft pass (layer l's attention waits for ev_ctx[l])
    float *part_c = nullptr, *sumsq_c = nullptr;
    uint8_t* acts_hc = nullptr;
    cudaStream_t st_side = nullptr;
    cudaEvent_t ev_ctx[DFL_MAX_DRAFTER_LAYERS] = {};
    // one-shot hook called when a draft pass has been queued (before anyone waits for it): the outer loop uses it to
    // queue the target's rollback behind the drafter's launches instead of in front of them
    void (*after_enqueue)(void*) = nullptr;
    void* after_enqueue_arg = nullptr;
    int32_t* pinned_i = nullptr;
    cudaStream_t st = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    int* err = nullptr;
    std::vector<void*> allocs;
};

namespace dfl {
dfl_status dsession_project_pending(dfl_dsession* ds, bool on_side = false);
dfl_status dsession_append_dev(dfl_dsession* ds, const float* rows_dev, cudaMemcpyKind kind, const uint32_t* positions, uint32_t count);
}

extern "C" {

dfl_status dfl_drafter_create(const dfl_model* target, const dfl_dflash_config* cfg, const dfl_tensor* tensors, uint64_t n_tensors,
                              dfl_drafter** out) {
    if (!target || !cfg || !tensors || !out) return fail(DFL_ERR_BAD_ARG, "drafter_create: null argument");
    *out = nullptr;
    DFL_CHECK(use_device(target->device));
    const dfl_dflash_config& c = *cfg;
    if (c.hidden_size != target->arch.hidden_size) return fail(DFL_ERR_BAD_SHAPE, "drafter requires H_drafter == H_target");
    if (c.n_layer == 0 || c.n_layer > DFL_MAX_DRAFTER_LAYERS) return fail(DFL_ERR_BAD_SHAPE, "drafter_create: layer count");
    if (c.block_size < 1 || c.block_size > MAX_ROWS) return fail(DFL_ERR_BAD_SHAPE, "drafter_create: block_size must be in [1, 16]");
    if (c.n_target_layers < 1 || c.n_target_layers > DFL_MAX_TARGET_LAYERS) return fail(DFL_ERR_BAD_SHAPE, "drafter_create: target layer count");
    if (c.head_dim != 128 && c.head_dim != 256) return fail(DFL_ERR_UNSUPPORTED, "drafter_create: head_dim must be 128 or 256");
    if (c.n_kv_heads == 0 || c.n_q_heads % c.n_kv_heads || ((uint64_t)c.n_q_heads * c.head_dim) % 256 || c.intermediate_size % 256)
        return fail(DFL_ERR_BAD_SHAPE, "drafter_create: head counts / widths");
    if (c.mask_token_id < 0 || (uint32_t)c.mask_token_id >= target->arch.vocab_size) return fail(DFL_ERR_BAD_TOKEN, "drafter_create: mask token id");
    for (uint32_t k = 0; k < c.n_target_layers; ++k)
        if (c.target_layer_ids[k] >= target->arch.n_layer) return fail(DFL_ERR_BAD_SHAPE, "drafter_create: target layer id out of range");
    TensorMap tm;
    for (uint64_t i = 0; i < n_tensors; ++i) {
        if (!tensors[i].name || !tensors[i].data) return fail(DFL_ERR_BAD_ARG, "drafter_create: tensor without name or data");
        tm.t[tensors[i].name] = &tensors[i];
    }
    auto* d = new dfl_drafter();
    d->target = target;
    d->cfg = c;
    const int dev = target->device;
    const uint64_t H = c.hidden_size, F = c.intermediate_size, q_dim = (uint64_t)c.n_q_heads * c.head_dim, kv_dim = (uint64_t)c.n_kv_heads * c.head_dim;
    const uint64_t KH = (uint64_t)c.n_target_layers * H;
    dfl_status s = DFL_OK;
    auto blk = [](uint32_t il, const char* suffix) { return "blk." + std::to_string(il) + "." + suffix; };
#define DC(expr)                      \
    do {                              \
        s = (expr);                   \
        if (s != DFL_OK) goto failed; \
    } while (0)
    DC(build_group(dev, 0, tm, {"dflash_fc.weight"}, KH, {H}, &d->fc, true));
    DC(upload_f32(dev, 0, tm, "dflash_hidden_norm.weight", H, &d->hidden_norm_w));
    DC(upload_f32(dev, 0, tm, "output_norm.weight", H, &d->out_norm_w));
    d->weight_bytes = d->fc.ggml_bytes();
    d->layers.resize(c.n_layer);
    for (uint32_t il = 0; il < c.n_layer; ++il) {
        DLayerW& L = d->layers[il];
        L.is_swa = c.layer_is_swa[il] != 0;
        DC(upload_f32(dev, 0, tm, blk(il, "attn_norm.weight"), H, &L.attn_norm_w));
        DC(upload_f32(dev, 0, tm, blk(il, "post_attention_norm.weight"), H, &L.post_norm_w));
        DC(upload_f32(dev, 0, tm, blk(il, "attn_q_norm.weight"), c.head_dim, &L.q_norm_w));
        DC(upload_f32(dev, 0, tm, blk(il, "attn_k_norm.weight"), c.head_dim, &L.k_norm_w));
        DC(build_group(dev, 0, tm, {blk(il, "attn_q.weight"), blk(il, "attn_k.weight"), blk(il, "attn_v.weight")}, H, {q_dim, kv_dim, kv_dim}, &L.qkv, true));
        DC(build_group(dev, 0, tm, {blk(il, "attn_k.weight"), blk(il, "attn_v.weight")}, H, {kv_dim, kv_dim}, &L.kv, true));
        DC(build_group(dev, 0, tm, {blk(il, "attn_output.weight")}, q_dim, {H}, &L.wo, true));
        DC(build_group(dev, 0, tm, {blk(il, "ffn_gate.weight"), blk(il, "ffn_up.weight")}, H, {F, F}, &L.gate_up, true));
        DC(build_group(dev, 0, tm, {blk(il, "ffn_down.weight")}, F, {H}, &L.down, true));
        d->weight_bytes += L.qkv.ggml_bytes() + L.wo.ggml_bytes() + L.gate_up.ggml_bytes() + L.down.ggml_bytes();
    }
    if (c.selector_rank > 0) {   // MetalDFlashHead::load, metal_dflash.rs:5008-5036
        if (c.selector_top_k != 16) { s = fail(DFL_ERR_UNSUPPORTED, "only selector_top_k=16 is supported"); goto failed; }
        DC(build_group(dev, 0, tm, {"selector_hidden.weight"}, H, {(uint64_t)c.selector_rank}, &d->sel_hidden, true));
        for (int which = 0; which < 2; ++which) {
            const char* name = which ? "selector_successor.weight" : "selector_predecessor.weight";
            auto it = tm.t.find(name);
            if (it == tm.t.end()) { s = fail(DFL_ERR_MISSING_TENSOR, std::string("missing tensor ") + name); goto failed; }
            const dfl_tensor& t = *it->second;
            if (t.on_device) { s = fail(DFL_ERR_BAD_ARG, "selector codebooks must be passed as host tensors"); goto failed; }
            if (t.n_dims != 2 || t.shape[0] != c.selector_rank) { s = fail(DFL_ERR_BAD_SHAPE, "selector codebook must be [rank, vocab]"); goto failed; }
            DC(dfl_codebook_create(t.dtype, t.shape[0], t.shape[1], t.data, t.n_bytes, which ? &d->sel_succ : &d->sel_pred));
        }
        d->has_selector = true;
        d->weight_bytes += d->sel_hidden.ggml_bytes();
    }
#undef DC
    d->weight_bytes += target->lm_head.ggml_bytes();
    cudaDeviceSynchronize();
    *out = d;
    return DFL_OK;
failed:
    dfl_drafter_destroy(d);
    return s;
}

void dfl_drafter_destroy(dfl_drafter* d) {
    if (!d) return;
    cudaSetDevice(d->target->device);
    d->fc.release();
    for (auto& L : d->layers) {
        L.qkv.release(); L.kv.release(); L.wo.release(); L.gate_up.release(); L.down.release();
        for (float* p : {L.attn_norm_w, L.post_norm_w, L.q_norm_w, L.k_norm_w})
            if (p) cudaFree(p);
    }
    if (d->hidden_norm_w) cudaFree(d->hidden_norm_w);
    if (d->out_norm_w) cudaFree(d->out_norm_w);
    d->sel_hidden.release();
    dfl_codebook_destroy(d->sel_pred);
    dfl_codebook_destroy(d->sel_succ);
    delete d;
}

uint64_t dfl_drafter_weight_bytes(const dfl_drafter* d) { return d ? d->weight_bytes : 0; }

dfl_status dfl_dsession_create(const dfl_drafter* d, uint32_t ctx_capacity, dfl_dsession** out) {
    if (!d || !out) return fail(DFL_ERR_BAD_ARG, "dsession_create: null argument");
    *out = nullptr;
    if (ctx_capacity == 0) return fail(DFL_ERR_BAD_ARG, "dsession_create: ctx_capacity must be positive");
    DFL_CHECK(use_device(d->target->device));
    auto* ds = new dfl_dsession();
    ds->d = d;
    ds->ctx_capacity = ctx_capacity;
    const dfl_dflash_config& c = d->cfg;
    const uint64_t H = c.hidden_size, F = c.intermediate_size, V = d->target->arch.vocab_size;
    const uint64_t q_dim = (uint64_t)c.n_q_heads * c.head_dim, kv_dim = (uint64_t)c.n_kv_heads * c.head_dim, KH = (uint64_t)c.n_target_layers * H;
    uint64_t part = 0;
    auto upd = [&](const MatGroup& g) { part = std::max<uint64_t>(part, (uint64_t)g.splits * MAX_ROWS * g.total_cols); };
    upd(d->fc);
    for (auto& L : d->layers) { upd(L.qkv); upd(L.kv); upd(L.wo); upd(L.gate_up); upd(L.down); }
    if (d->target->lm_head.splits > 1) upd(d->target->lm_head);
    if (d->has_selector) upd(d->sel_hidden);
    bool ok = cudaStreamCreateWithFlags(&ds->st, cudaStreamNonBlocking) == cudaSuccess;
    auto alloc = [&](size_t bytes) -> void* {
        if (!ok) return nullptr;
        void* q = nullptr;
        ok = cudaMalloc(&q, bytes ? bytes : 16) == cudaSuccess;
        if (ok) { cudaMemset(q, 0, bytes ? bytes : 16); ds->allocs.push_back(q); }
        return q;
    };
    const AttnGeom g = d->geom((int)c.n_q_heads);
    ds->staging = (float*)alloc((size_t)kPendingCap * KH * 4);
    ds->pos_ctx_dev = (uint32_t*)alloc(((size_t)ctx_capacity + KV_TILE_KEYS) / KV_TILE_KEYS * KV_TILE_KEYS * 4);   // whole tiles of positions are staged
    // Tiled shadow (tcgen05 attention) for the layers that attend over the whole context, where scanning it is what the
    // draft pass spends its time on: contexts of 16384 columns and more, 128-wide heads in groups of four.
    // DFL_DATTN_TILED=1 / 0 forces it on (where the geometry fits) or off.
    bool tiled = false;
    if (c.head_dim == 128 && c.n_kv_heads && c.n_q_heads / c.n_kv_heads == 4 && c.n_q_heads % c.n_kv_heads == 0) {
        const char* e = getenv("DFL_DATTN_TILED");
        tiled = e ? e[0] == '1' : ctx_capacity >= 16384;
    }
    for (uint32_t il = 0; il < c.n_layer; ++il) {
        ds->k_ctx.push_back((float*)alloc((size_t)ctx_capacity * kv_dim * 4));
        ds->v_ctx.push_back((float*)alloc((size_t)ctx_capacity * kv_dim * 4));
        const bool full_layer = !(c.layer_is_swa[il] && c.swa_window > 0);
        ds->ctx_tiles.push_back(tiled && full_layer ? alloc(dattn_t5_tile_halfs((int)c.n_kv_heads, ctx_capacity) * 2) : nullptr);
    }
    if (tiled) ds->noise_tiles = alloc(dattn_t5_tile_halfs((int)c.n_kv_heads, MAX_ROWS) * 2);
    ds->x = (float*)alloc(MAX_ROWS * H * 4);
    ds->part = (float*)alloc(part * 4);
    ds->sumsq = (float*)alloc((H / GLUE_COLS) * MAX_ROWS * 4);
    ds->q_rot = (float*)alloc(MAX_ROWS * q_dim * 4);
    ds->k_noise = (float*)alloc(MAX_ROWS * kv_dim * 4);
    ds->v_noise = (float*)alloc(MAX_ROWS * kv_dim * 4);
    ds->attn_part = (float*)alloc(attn_partials_floats(g, (ctx_capacity + KV_TILE_KEYS - 1) / KV_TILE_KEYS * KV_TILE_KEYS + 2 * KV_TILE_KEYS) * 4);   // also two records per tile of the tiled path, the block's own tile included
    ds->acts_h = (uint8_t*)alloc(acts_bytes(DFL_BF16, H));
    ds->acts_f = (uint8_t*)alloc(acts_bytes(DFL_BF16, F));
    ds->acts_q = (uint8_t*)alloc(acts_bytes(DFL_BF16, q_dim));
    ds->acts_fc = (uint8_t*)alloc(acts_bytes(DFL_BF16, KH));
    {
        uint64_t part_c = (uint64_t)d->fc.splits * MAX_ROWS * d->fc.total_cols;
        for (auto& L : d->layers) part_c = std::max<uint64_t>(part_c, (uint64_t)L.kv.splits * MAX_ROWS * L.kv.total_cols);
        ds->part_c = (float*)alloc(part_c * 4);
        ds->sumsq_c = (float*)alloc((H / GLUE_COLS) * MAX_ROWS * 4);
        ds->acts_hc = (uint8_t*)alloc(acts_bytes(DFL_BF16, H));
    }
    ds->acts_lm = (uint8_t*)alloc(acts_bytes(DFL_BF16, H));
    ds->logits = (float*)alloc(MAX_ROWS * V * 4);
    ds->gap = (float*)alloc(MAX_ROWS * 4);
    ds->argmax = (int32_t*)alloc(MAX_ROWS * 4);
    ds->tokens_dev = (int32_t*)alloc(MAX_ROWS * 4);
    ds->am_scratch = alloc(MAX_ROWS * ARGMAX_PARTS * 16);
    ds->topk_ids = (int32_t*)alloc(MAX_ROWS * 16 * 4);
    ds->topk_vals = (float*)alloc(MAX_ROWS * 16 * 4);
    ds->topk_scratch = alloc(topk16_scratch_bytes(MAX_ROWS));
    if (d->has_selector) {
        ds->sel_h = (float*)alloc((size_t)MAX_ROWS * c.selector_rank * 4);
        ds->acts_sel = (uint8_t*)alloc(acts_bytes(DFL_BF16, H));
    }
    ds->err = (int*)alloc(4);
    ok = ok && cudaMallocHost(&ds->pinned_i, 2 * MAX_ROWS * 4) == cudaSuccess;
    ok = ok && cudaMallocHost(&ds->pinned_sel, MAX_ROWS * 16 * 8 + (size_t)MAX_ROWS * c.selector_rank * 4) == cudaSuccess;
    ok = ok && cudaEventCreate(&ds->ev0) == cudaSuccess && cudaEventCreate(&ds->ev1) == cudaSuccess;
    ok = ok && cudaStreamCreateWithFlags(&ds->st_side, cudaStreamNonBlocking) == cudaSuccess;
    for (uint32_t il = 0; il < c.n_layer; ++il) ok = ok && cudaEventCreateWithFlags(&ds->ev_ctx[il], cudaEventDisableTiming) == cudaSuccess;
    if (!ok) {
        std::string why = cudaGetErrorString(cudaGetLastError());
        dfl_dsession_destroy(ds);
        return fail(DFL_ERR_OOM, "dsession_create: allocation failed: " + why);
    }
    ds->pos_host.reserve(ctx_capacity);
    cudaDeviceSynchronize();
    *out = ds;
    return DFL_OK;
}

void dfl_dsession_destroy(dfl_dsession* ds) {
    if (!ds) return;
    cudaSetDevice(ds->d->target->device);
    for (void* p : ds->allocs) cudaFree(p);
    if (ds->pinned_i) cudaFreeHost(ds->pinned_i);
    if (ds->pinned_sel) cudaFreeHost(ds->pinned_sel);
    if (ds->ev0) cudaEventDestroy(ds->ev0);
    if (ds->ev1) cudaEventDestroy(ds->ev1);
    for (auto& e : ds->ev_ctx)
        if (e) cudaEventDestroy(e);
    if (ds->st_side) cudaStreamDestroy(ds->st_side);
    if (ds->st) cudaStreamDestroy(ds->st);
    delete ds;
}

uint32_t dfl_dsession_ctx_len(const dfl_dsession* ds) { return ds ? ds->ctx_len : 0; }

// Internal view for the outer loop (generate.cu); not part of the public header.
struct dfl_dsession_view {
    cudaStream_t st;
    cudaEvent_t ev0, ev1;
    int* err;
    const int32_t* argmax_dev;
    const float* logits_dev;
    int32_t* pinned_i;
    uint32_t block_size, n_target_layers;
    const uint32_t* target_layer_ids;
    const dfl_model* target;
    int32_t has_selector;
};
void dfl_dsession_view_get(dfl_dsession* ds, dfl_dsession_view* out) {
    out->st = ds->st; out->ev0 = ds->ev0; out->ev1 = ds->ev1; out->err = ds->err;
    out->argmax_dev = ds->argmax; out->logits_dev = ds->logits; out->pinned_i = ds->pinned_i;
    out->has_selector = ds->d->has_selector ? 1 : 0;
    out->block_size = ds->d->cfg.block_size; out->n_target_layers = ds->d->cfg.n_target_layers;
    out->target_layer_ids = ds->d->cfg.target_layer_ids; out->target = ds->d->target;
}

dfl_status dfl_dsession_reset(dfl_dsession* ds) {
    if (!ds) return fail(DFL_ERR_BAD_ARG, "dsession_reset: null session");
    ds->ctx_len = ds->ready = ds->pending_base = 0;
    ds->pos_host.clear();
    return DFL_OK;
}

}  // extern "C"

namespace dfl {

// Projects every appended-but-unprojected column: fc + hidden_norm, then per layer K/V + K-norm + RoPE.  With on_side
// the work goes to the session's side stream and layer l's rows are complete when ev_ctx[l] fires (recorded after the
// last block of columns); its scratch is separate from the draft pass's, the rows it writes are beyond every row a
// running attention reads.
dfl_status dsession_project_pending(dfl_dsession* ds, bool on_side) {
    const dfl_drafter* d = ds->d;
    const dfl_dflash_config& c = d->cfg;
    const uint64_t H = c.hidden_size, KH = (uint64_t)c.n_target_layers * H;
    cudaStream_t st = on_side ? ds->st_side : ds->st;
    GemmEpilogue ep_norm;
    ep_norm.sumsq = ds->sumsq_c;
    ep_norm.n_sumsq = (int)(H / GLUE_COLS);
    ep_norm.norm_k = (float)H;
    ep_norm.eps = c.rms_norm_eps;
    const AttnGeom gkv = d->geom(0);
    while (ds->ready < ds->ctx_len) {
        const uint32_t c0 = ds->ready, nb = std::min<uint32_t>(MAX_ROWS, ds->ctx_len - c0);
        const bool last_block = c0 + nb == ds->ctx_len;
        GlueParams p;
        p.mode = GLUE_COPY;
        p.x = ds->staging + (uint64_t)(c0 - ds->pending_base) * KH;
        p.ld_x = (int)KH;
        p.acts = ds->acts_fc; p.bf3 = act_layout_of(d->fc.mats[0]);
        p.n_rows = (int)nb; p.err = ds->err;
        DFL_CHECK(launch_glue(st, p, KH));
        DFL_CHECK(launch_group(st, d->fc, ds->acts_fc, ds->part_c, GemmEpilogue{}, ds->err));
        GlueParams q;
        q.mode = GLUE_RESID;
        q.part = ds->part_c; q.splits = d->fc.splits; q.ld_part = (int)d->fc.total_cols;
        q.mul_w = d->hidden_norm_w;
        q.sumsq = ds->sumsq_c;
        q.acts = ds->acts_hc; q.bf3 = act_layout_of(d->layers[0].kv.mats[0]);
        q.n_rows = (int)nb; q.err = ds->err;
        DFL_CHECK(launch_glue(st, q, H));
        for (uint32_t il = 0; il < c.n_layer; ++il) {
            const DLayerW& L = d->layers[il];
            DFL_CHECK(launch_group(st, L.kv, ds->acts_hc, ds->part_c, ep_norm, ds->err));
            DFL_CHECK(launch_attn_front(st, gkv, false, ds->part_c, L.kv.splits, (int)L.kv.total_cols, nullptr, L.k_norm_w, 0, (int)nb, ds->k_ctx[il],
                                        ds->v_ctx[il], KV_F32_ROWS, nullptr, nullptr, ds->pos_ctx_dev + c0, (long long)c0));
            if (ds->ctx_tiles[il]) DFL_CHECK(launch_dctx_tiles(st, ds->k_ctx[il], ds->v_ctx[il], (int)c.n_kv_heads, c0, nb, c0, ds->ctx_tiles[il]));
            if (on_side && last_block) DFL_CUDA(cudaEventRecord(ds->ev_ctx[il], st));
        }
        ds->ready += nb;
    }
    ds->pending_base = ds->ready;
    return DFL_OK;
}

dfl_status dsession_append_dev(dfl_dsession* ds, const float* rows, cudaMemcpyKind kind, const uint32_t* positions, uint32_t count) {
    const dfl_dflash_config& c = ds->d->cfg;
    const uint64_t KH = (uint64_t)c.n_target_layers * c.hidden_size;
    if ((uint64_t)ds->ctx_len + count > ds->ctx_capacity)
        return fail(DFL_ERR_CTX_OVERFLOW, "drafter context is full: " + std::to_string(ds->ctx_len) + " + " + std::to_string(count) + " > " +
                                              std::to_string(ds->ctx_capacity));
    uint32_t done = 0;
    while (done < count) {
        if (ds->ctx_len - ds->pending_base >= kPendingCap) DFL_CHECK(dsession_project_pending(ds));
        const uint32_t room = kPendingCap - (ds->ctx_len - ds->pending_base);
        const uint32_t nb = std::min(room, count - done);
        DFL_CUDA(cudaMemcpyAsync(ds->staging + (uint64_t)(ds->ctx_len - ds->pending_base) * KH, rows + (uint64_t)done * KH, (size_t)nb * KH * 4, kind, ds->st));
        for (uint32_t i = 0; i < nb; ++i) ds->pos_host.push_back(positions[done + i]);
        DFL_CUDA(cudaMemcpyAsync(ds->pos_ctx_dev + ds->ctx_len, ds->pos_host.data() + ds->ctx_len, (size_t)nb * 4, cudaMemcpyHostToDevice, ds->st));
        // pos_host may reallocate later: the copy above must finish first
        DFL_CUDA(cudaStreamSynchronize(ds->st));
        ds->ctx_len += nb;
        done += nb;
    }
    return DFL_OK;
}

// ---- drafter context in a session snapshot -----------------------------------------------------------------------
// What a restored request needs of the drafter is the context it can still see: every column when a layer has full
// attention, else the last `swa_window` columns (dflash_capture_window_limit, metal_dflash.rs:110-118).  The reference
// stores those columns raw (K * H f32 each) and projects them again on restore; this library stores their projected,
// rotated K / V rows (half the bytes, nothing to recompute), which are exactly what the attention kernels read.
uint32_t dsession_tail_columns(const dfl_dsession* ds) {
    const dfl_dflash_config& c = ds->d->cfg;
    bool all_swa = c.swa_window > 0;
    for (uint32_t il = 0; il < c.n_layer; ++il) all_swa = all_swa && c.layer_is_swa[il] != 0;
    return all_swa ? std::min(ds->ctx_len, c.swa_window) : ds->ctx_len;
}
uint64_t dsession_snapshot_bytes(const dfl_dsession* ds) {
    const dfl_dflash_config& c = ds->d->cfg;
    const uint64_t cols = dsession_tail_columns(ds), kv_dim = (uint64_t)c.n_kv_heads * c.head_dim;
    return cols * 4 + (uint64_t)c.n_layer * 2 * cols * kv_dim * 4;
}
// layout: positions u32[cols], then per layer K rows [cols][kv_dim] f32 and V rows [cols][kv_dim] f32
dfl_status dsession_snapshot_write(dfl_dsession* ds, uint8_t* dst, uint32_t* cols_out) {
    DFL_CHECK(dsession_project_pending(ds));
    const dfl_dflash_config& c = ds->d->cfg;
    const uint32_t cols = dsession_tail_columns(ds), first = ds->ctx_len - cols;
    const uint64_t kv_dim = (uint64_t)c.n_kv_heads * c.head_dim, rows = (uint64_t)cols * kv_dim * 4;
    memcpy(dst, ds->pos_host.data() + first, (size_t)cols * 4);
    dst += (size_t)cols * 4;
    for (uint32_t il = 0; il < c.n_layer && cols; ++il) {
        DFL_CUDA(cudaMemcpyAsync(dst, ds->k_ctx[il] + (uint64_t)first * kv_dim, rows, cudaMemcpyDeviceToHost, ds->st));
        DFL_CUDA(cudaMemcpyAsync(dst + rows, ds->v_ctx[il] + (uint64_t)first * kv_dim, rows, cudaMemcpyDeviceToHost, ds->st));
        dst += 2 * rows;
    }
    DFL_CHECK(check_dev_err(ds->st, ds->err));
    *cols_out = cols;
    return DFL_OK;
}
// what a drafter section depends on besides its column count: layer count, K/V row width, window
void dsession_identity(const dfl_dsession* ds, uint32_t out[3]) {
    const dfl_dflash_config& c = ds->d->cfg;
    out[0] = c.n_layer;
    out[1] = c.n_kv_heads * c.head_dim;
    out[2] = c.swa_window;
}
dfl_status dsession_snapshot_validate(const dfl_dsession* ds, uint32_t cols, uint64_t n_bytes) {
    const dfl_dflash_config& c = ds->d->cfg;
    const uint64_t kv_dim = (uint64_t)c.n_kv_heads * c.head_dim, rows = (uint64_t)cols * kv_dim * 4;
    if (cols > ds->ctx_capacity) return fail(DFL_ERR_CTX_OVERFLOW, "snapshot: drafter context tail exceeds the session's capacity");
    if (n_bytes != (uint64_t)cols * 4 + (uint64_t)c.n_layer * 2 * rows) return fail(DFL_ERR_BAD_SHAPE, "snapshot: drafter section length mismatch");
    return DFL_OK;
}
dfl_status dsession_snapshot_read(dfl_dsession* ds, const uint8_t* src, uint32_t cols, uint64_t n_bytes) {
    const dfl_dflash_config& c = ds->d->cfg;
    const uint64_t kv_dim = (uint64_t)c.n_kv_heads * c.head_dim, rows = (uint64_t)cols * kv_dim * 4;
    DFL_CHECK(dsession_snapshot_validate(ds, cols, n_bytes));
    ds->ctx_len = ds->ready = ds->pending_base = 0;
    ds->pos_host.assign(reinterpret_cast<const uint32_t*>(src), reinterpret_cast<const uint32_t*>(src) + cols);
    if (cols) DFL_CUDA(cudaMemcpyAsync(ds->pos_ctx_dev, ds->pos_host.data(), (size_t)cols * 4, cudaMemcpyHostToDevice, ds->st));
    src += (size_t)cols * 4;
    for (uint32_t il = 0; il < c.n_layer && cols; ++il) {
        DFL_CUDA(cudaMemcpyAsync(ds->k_ctx[il], src, rows, cudaMemcpyHostToDevice, ds->st));
        DFL_CUDA(cudaMemcpyAsync(ds->v_ctx[il], src + rows, rows, cudaMemcpyHostToDevice, ds->st));
        if (ds->ctx_tiles[il]) DFL_CHECK(launch_dctx_tiles(ds->st, ds->k_ctx[il], ds->v_ctx[il], (int)c.n_kv_heads, 0, cols, 0, ds->ctx_tiles[il]));
        src += 2 * rows;
    }
    DFL_CUDA(cudaStreamSynchronize(ds->st));
    ds->ctx_len = ds->ready = ds->pending_base = cols;
    return DFL_OK;
}
const dfl_model* dsession_target(const dfl_dsession* ds) { return ds->d->target; }

// One draft pass; leaves logits / argmax on the device, and with `topk` (always on a drafter with a selector) the
// top-16 per row plus the selector's gate rows (phase-4 tail, metal_dflash.rs:17099-17128).
dfl_status draft_core(dfl_dsession* ds, int32_t carry, uint32_t noise_start, bool topk) {
    const dfl_drafter* d = ds->d;
    const dfl_model* tgt = d->target;
    const dfl_dflash_config& c = d->cfg;
    const uint64_t H = c.hidden_size, F = c.intermediate_size, V = tgt->arch.vocab_size;
    const int n = (int)c.block_size;
    cudaStream_t st = ds->st;
    // the columns appended since the last pass are projected on the side stream while this pass starts
    // (DFL_SIDE_STREAM=0: before it, on the same stream)
    static const bool side_enabled = [] { const char* e = getenv("DFL_SIDE_STREAM"); return !(e && e[0] == '0'); }();
    const bool ctx_on_side = side_enabled && ds->ready < ds->ctx_len;
    if (ctx_on_side) {   // order the side stream after everything this session has queued on its main stream
        DFL_CUDA(cudaEventRecord(ds->ev1, st));
        DFL_CUDA(cudaStreamWaitEvent(ds->st_side, ds->ev1, 0));
    }
    DFL_CHECK(dsession_project_pending(ds, ctx_on_side));
    GemmEpilogue ep_norm;
    ep_norm.sumsq = ds->sumsq;
    ep_norm.n_sumsq = (int)(H / GLUE_COLS);
    ep_norm.norm_k = (float)H;
    ep_norm.eps = c.rms_norm_eps;
    ds->pinned_i[0] = carry;
    for (int i = 1; i < n; ++i) ds->pinned_i[i] = c.mask_token_id;
    DFL_CUDA(cudaMemcpyAsync(ds->tokens_dev, ds->pinned_i, n * 4, cudaMemcpyHostToDevice, st));
    DFL_CHECK(launch_embed_rows(st, tgt->embd_dtype, tgt->embd_ggml, H, ds->tokens_dev, n, ds->x, (int)H));
    auto norm_glue = [&](const float* part, int splits, int ld_part, const float* w, uint8_t* acts, int layout) -> dfl_status {
        GlueParams p;
        p.mode = GLUE_RESID;
        p.part = part; p.splits = splits; p.ld_part = ld_part;
        p.x = ds->x; p.ld_x = (int)H;
        p.mul_w = w;
        p.acts = acts; p.bf3 = layout;
        p.sumsq = ds->sumsq;
        p.n_rows = n; p.err = ds->err;
        return launch_glue(st, p, H);
    };
    auto bf = [](const MatGroup& g) { return act_layout_of(g.mats[0]); };
    DFL_CHECK(norm_glue(nullptr, 0, 0, d->layers[0].attn_norm_w, ds->acts_h, bf(d->layers[0].qkv)));
    const AttnGeom g = d->geom((int)c.n_q_heads);
    // context columns an all-SWA layer can see start at the first position >= noise_start - (window - 1)
    bool monotonic = true;
    for (size_t i = 1; i < ds->pos_host.size() && monotonic; ++i) monotonic = ds->pos_host[i] >= ds->pos_host[i - 1];
    for (uint32_t il = 0; il < c.n_layer; ++il) {
        const DLayerW& L = d->layers[il];
        DFL_CHECK(launch_group(st, L.qkv, ds->acts_h, ds->part, ep_norm, ds->err));
        DFL_CHECK(launch_attn_front(st, g, false, ds->part, L.qkv.splits, (int)L.qkv.total_cols, L.q_norm_w, L.k_norm_w, noise_start, n, ds->k_noise,
                                    ds->v_noise, KV_F32_ROWS, ds->q_rot, nullptr, nullptr, 0));
        const uint32_t window = L.is_swa ? c.swa_window : 0;
        int ctx_begin = 0;
        if (window > 0 && monotonic) {  // dflash_swa_ctx_scan_start, metal_dflash.rs:570-594
            const uint32_t min_pos = noise_start >= window - 1 ? noise_start - (window - 1) : 0;
            ctx_begin = (int)(std::lower_bound(ds->pos_host.begin(), ds->pos_host.begin() + ds->ctx_len, min_pos) - ds->pos_host.begin());
        }
        if (ctx_on_side) DFL_CUDA(cudaStreamWaitEvent(st, ds->ev_ctx[il], 0));
        if (ds->ctx_tiles[il] && window == 0) {
            // the whole context through the tcgen05 kernel: the block's own rows become one more tile set first
            int n_records = 0;
            DFL_CHECK(launch_dctx_tiles(st, ds->k_noise, ds->v_noise, (int)c.n_kv_heads, 0, (uint32_t)n, 0, ds->noise_tiles));
            DFL_CHECK(launch_dattn_t5(st, g, ds->q_rot, ds->ctx_tiles[il], ds->noise_tiles, ds->pos_ctx_dev, (int)ds->ctx_len, noise_start, n,
                                      c.causal != 0, ds->attn_part, ds->ctx_capacity, ds->err, &n_records));
            DFL_CHECK(launch_dattn_post(st, g, ds->attn_part, n_records, n, ds->acts_q, bf(L.wo), ds->err));
        } else
        DFL_CHECK(launch_drafter_attn(st, g, ds->q_rot, ds->k_ctx[il], ds->v_ctx[il], reinterpret_cast<const int32_t*>(ds->pos_ctx_dev), ctx_begin,
                                      (int)ds->ctx_len, ds->k_noise, ds->v_noise, noise_start, n, c.causal != 0, window, ds->attn_part, ds->acts_q,
                                      bf(L.wo), ds->err,
                                      // span length follows the keys the layer can see: a sliding-window layer over a
                                      // monotonic context never scans more than window - 1 + n keys
                                      window > 0 && monotonic ? std::min<uint32_t>(ds->ctx_capacity, window - 1 + (uint32_t)n) : ds->ctx_capacity));
        DFL_CHECK(launch_group(st, L.wo, ds->acts_q, ds->part, GemmEpilogue{}, ds->err));
        DFL_CHECK(norm_glue(ds->part, L.wo.splits, (int)L.wo.total_cols, L.post_norm_w, ds->acts_h, bf(L.gate_up)));
        DFL_CHECK(launch_group(st, L.gate_up, ds->acts_h, ds->part, ep_norm, ds->err));
        GlueParams p;
        p.mode = GLUE_SWIGLU;
        p.part = ds->part; p.splits = L.gate_up.splits; p.ld_part = (int)L.gate_up.total_cols;
        p.swiglu_f = (int)F;
        const int down_layout = bf(L.down);
        const bool down_bf = down_layout == ACT_BF3 || down_layout == ACT_TSB;
        p.pre_scale = down_bf ? 1.0f : 1.0f / 64.0f;
        p.acts = ds->acts_f; p.bf3 = down_layout;
        p.n_rows = n; p.err = ds->err;
        DFL_CHECK(launch_glue(st, p, F));
        GemmEpilogue ep_down;
        ep_down.out_scale = down_bf ? 1.0f : 64.0f;
        DFL_CHECK(launch_group(st, L.down, ds->acts_f, ds->part, ep_down, ds->err));
        const bool last = il + 1 == c.n_layer;
        if (last) DFL_CHECK(norm_glue(ds->part, L.down.splits, (int)L.down.total_cols, d->out_norm_w, ds->acts_lm, bf(tgt->lm_head)));
        else DFL_CHECK(norm_glue(ds->part, L.down.splits, (int)L.down.total_cols, d->layers[il + 1].attn_norm_w, ds->acts_h, bf(d->layers[il + 1].qkv)));
    }
    const MatGroup& lm = tgt->lm_head;
    if (lm.splits == 1) {
        DFL_CHECK(launch_group(st, lm, ds->acts_lm, ds->logits, ep_norm, ds->err));
        DFL_CHECK(launch_argmax_top2(st, ds->logits, n, V, V, ds->argmax, ds->gap, ds->am_scratch));
    } else {
        DFL_CHECK(launch_group(st, lm, ds->acts_lm, ds->part, ep_norm, ds->err));
        DFL_CHECK(launch_reduce_argmax_top2(st, ds->part, lm.splits, n, V, ds->logits, V, ds->argmax, ds->gap, ds->am_scratch));
    }
    ds->have_topk = false;
    if (topk || d->has_selector) {
        DFL_CHECK(launch_topk16(st, ds->logits, n, V, V, ds->topk_ids, ds->topk_vals, ds->topk_scratch));
        if (d->has_selector) {
            const MatGroup& sh = d->sel_hidden;
            const uint8_t* acts = ds->acts_lm;
            if (bf(sh) != bf(lm)) {   // the normalised hidden again, packed for this matrix's kernel family
                DFL_CHECK(norm_glue(nullptr, 0, 0, d->out_norm_w, ds->acts_sel, bf(sh)));
                acts = ds->acts_sel;
            }
            if (sh.splits == 1) {
                DFL_CHECK(launch_group(st, sh, acts, ds->sel_h, ep_norm, ds->err));
            } else {
                DFL_CHECK(launch_group(st, sh, acts, ds->part, ep_norm, ds->err));
                DFL_CHECK(launch_reduce_partials(st, ds->part, sh.splits, n, c.selector_rank, ds->sel_h, (int)c.selector_rank));
            }
        }
        ds->have_topk = true;
    }
    if (ds->after_enqueue) {
        auto fn = ds->after_enqueue;
        ds->after_enqueue = nullptr;
        fn(ds->after_enqueue_arg);
    }
    return DFL_OK;
}
void dsession_set_after_enqueue(dfl_dsession* ds, void (*fn)(void*), void* arg) {
    ds->after_enqueue = fn;
    ds->after_enqueue_arg = arg;
}

// the last pass's top-16 and gate rows in pinned host memory (at most 18 KB; the reference reads the same three
// buffers after its wait, metal_dflash.rs:17184-17207)
struct SelectorHost {
    const int32_t* ids;
    const float *vals, *sel_h;
};
dfl_status selector_to_host(dfl_dsession* ds, SelectorHost* h) {
    const uint32_t n = ds->d->cfg.block_size, rank = ds->d->cfg.selector_rank;
    uint8_t* p = ds->pinned_sel;
    DFL_CUDA(cudaMemcpyAsync(p, ds->topk_ids, n * 16 * 4, cudaMemcpyDeviceToHost, ds->st));
    DFL_CUDA(cudaMemcpyAsync(p + MAX_ROWS * 16 * 4, ds->topk_vals, n * 16 * 4, cudaMemcpyDeviceToHost, ds->st));
    if (ds->d->has_selector) DFL_CUDA(cudaMemcpyAsync(p + MAX_ROWS * 16 * 8, ds->sel_h, (size_t)n * rank * 4, cudaMemcpyDeviceToHost, ds->st));
    DFL_CHECK(check_dev_err(ds->st, ds->err));
    h->ids = reinterpret_cast<const int32_t*>(p);
    h->vals = reinterpret_cast<const float*>(p + MAX_ROWS * 16 * 4);
    h->sel_h = reinterpret_cast<const float*>(p + MAX_ROWS * 16 * 8);
    return DFL_OK;
}

// per-row argmax drafts plus the top-16 of every row left on the device (for sparse proposals without a selector)
dfl_status draft_block_topk(dfl_dsession* ds, int32_t carry, uint32_t noise_start_pos, int32_t* out_tokens) {
    const dfl_model* tgt = ds->d->target;
    DFL_CHECK(use_device(tgt->device));
    if (carry < 0 || (uint32_t)carry >= tgt->arch.vocab_size) return fail(DFL_ERR_BAD_TOKEN, "draft_block: carry token out of range");
    const uint32_t n = ds->d->cfg.block_size;
    DFL_CHECK(draft_core(ds, carry, noise_start_pos, true));
    DFL_CUDA(cudaMemcpyAsync(ds->pinned_i + MAX_ROWS, ds->argmax, n * 4, cudaMemcpyDeviceToHost, ds->st));
    DFL_CHECK(check_dev_err(ds->st, ds->err));
    out_tokens[0] = carry;
    for (uint32_t i = 1; i < n; ++i) out_tokens[i] = ds->pinned_i[MAX_ROWS + i];
    return DFL_OK;
}

}  // namespace dfl

extern "C" {

dfl_status dfl_dsession_append_columns_host(dfl_dsession* ds, const float* cols_host, const uint32_t* positions, uint32_t count) {
    if (!ds || !cols_host || !positions) return fail(DFL_ERR_BAD_ARG, "append_columns: null argument");
    DFL_CHECK(use_device(ds->d->target->device));
    return dsession_append_dev(ds, cols_host, cudaMemcpyHostToDevice, positions, count);
}

dfl_status dfl_dsession_append_from_scratch(dfl_dsession* ds, const dfl_scratch* sc, uint32_t first_row, uint32_t count, uint32_t first_position) {
    if (!ds || !sc) return fail(DFL_ERR_BAD_ARG, "append_from_scratch: null argument");
    if (sc->m != ds->d->target) return fail(DFL_ERR_BAD_ARG, "append_from_scratch: scratch belongs to another model");
    if (sc->k_layers != ds->d->cfg.n_target_layers) return fail(DFL_ERR_BAD_SHAPE, "append_from_scratch: capture layer count differs from the drafter's");
    if (!sc->have_block || first_row + count > MAX_ROWS) return fail(DFL_ERR_BAD_SHAPE, "append_from_scratch: rows outside the captured block");
    DFL_CHECK(use_device(ds->d->target->device));
    uint32_t pos[MAX_ROWS];
    for (uint32_t i = 0; i < count; ++i) pos[i] = first_position + i;
    const uint64_t KH = (uint64_t)sc->k_layers * sc->m->arch.hidden_size;
    // the capture was written on the target session's stream, which the verify call has already synchronised
    return dsession_append_dev(ds, sc->capture + (uint64_t)first_row * KH, cudaMemcpyDeviceToDevice, pos, count);
}

dfl_status dfl_draft_block(dfl_dsession* ds, int32_t carry, uint32_t noise_start_pos, int32_t* out_tokens, float* logits_host) {
    if (!ds || !out_tokens) return fail(DFL_ERR_BAD_ARG, "draft_block: null argument");
    const dfl_model* tgt = ds->d->target;
    DFL_CHECK(use_device(tgt->device));
    if (carry < 0 || (uint32_t)carry >= tgt->arch.vocab_size) return fail(DFL_ERR_BAD_TOKEN, "draft_block: carry token out of range");
    const uint32_t n = ds->d->cfg.block_size;
    DFL_CHECK(draft_core(ds, carry, noise_start_pos, false));
    DFL_CUDA(cudaMemcpyAsync(ds->pinned_i + MAX_ROWS, ds->argmax, n * 4, cudaMemcpyDeviceToHost, ds->st));
    if (logits_host) DFL_CUDA(cudaMemcpyAsync(logits_host, ds->logits, (size_t)n * tgt->arch.vocab_size * 4, cudaMemcpyDeviceToHost, ds->st));
    if (ds->d->has_selector) {   // select_draft_path: the walk replaces the per-row argmax
        SelectorHost h;
        DFL_CHECK(selector_to_host(ds, &h));
        DFL_CHECK(dfl_selector_walk(ds->d->sel_pred, ds->d->sel_succ, 16, ds->d->cfg.selector_rank, carry, n, h.ids, h.vals, h.sel_h, out_tokens,
                                    nullptr, nullptr));
        out_tokens[0] = carry;
        return DFL_OK;
    }
    DFL_CHECK(check_dev_err(ds->st, ds->err));
    out_tokens[0] = carry;
    for (uint32_t i = 1; i < n; ++i) out_tokens[i] = ds->pinned_i[MAX_ROWS + i];
    return DFL_OK;
}

dfl_status dfl_draft_block_sampled(dfl_dsession* ds, int32_t carry, uint32_t noise_start_pos, dfl_sampler* proposal_sampler, int32_t* out_tokens,
                                   uint32_t* cand_offsets, int32_t* cand_tokens, double* cand_weights) {
    if (!ds || !proposal_sampler || !out_tokens || !cand_offsets || !cand_tokens || !cand_weights)
        return fail(DFL_ERR_BAD_ARG, "draft_block_sampled: null argument");
    if (!ds->d->has_selector) return fail(DFL_ERR_UNSUPPORTED, "sampled path requires a DFlash 2 selector");
    const dfl_model* tgt = ds->d->target;
    DFL_CHECK(use_device(tgt->device));
    if (carry < 0 || (uint32_t)carry >= tgt->arch.vocab_size) return fail(DFL_ERR_BAD_TOKEN, "draft_block: carry token out of range");
    dfl_sampling_config pc;
    dfl_sampler_get_config(proposal_sampler, &pc);
    if (!(pc.temperature > 0.0f) || pc.top_k != 0 || pc.top_p != 1.0f || pc.min_p != 0.0f)   // checked before any device work, :17279-17288
        return fail(DFL_ERR_SAMPLING, "DFlash 2 proposal sampler must use temperature without target filters");
    const uint32_t n = ds->d->cfg.block_size;
    DFL_CHECK(draft_core(ds, carry, noise_start_pos, true));
    SelectorHost h;
    DFL_CHECK(selector_to_host(ds, &h));
    DFL_CHECK(dfl_selector_walk_sampled(ds->d->sel_pred, ds->d->sel_succ, 16, ds->d->cfg.selector_rank, carry, n, h.ids, h.vals, h.sel_h,
                                        proposal_sampler, out_tokens, cand_offsets, cand_tokens, cand_weights));
    out_tokens[0] = carry;
    return DFL_OK;
}

dfl_status dfl_dsession_read_selector(dfl_dsession* ds, int32_t* ids_out, float* vals_out, float* sel_h_out) {
    if (!ds || !ids_out || !vals_out) return fail(DFL_ERR_BAD_ARG, "read_selector: null argument");
    if (!ds->have_topk) return fail(DFL_ERR_BAD_ARG, "read_selector: the last draft pass produced no top-16");
    if (sel_h_out && !ds->d->has_selector) return fail(DFL_ERR_UNSUPPORTED, "read_selector: the drafter has no selector");
    DFL_CHECK(use_device(ds->d->target->device));
    SelectorHost h;
    DFL_CHECK(selector_to_host(ds, &h));
    const uint32_t n = ds->d->cfg.block_size;
    memcpy(ids_out, h.ids, n * 16 * 4);
    memcpy(vals_out, h.vals, n * 16 * 4);
    if (sel_h_out) memcpy(sel_h_out, h.sel_h, (size_t)n * ds->d->cfg.selector_rank * 4);
    return DFL_OK;
}

}  // extern "C"
