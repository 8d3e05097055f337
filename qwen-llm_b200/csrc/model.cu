// Target model residency, per-sequence session, verify scratch and the packed verify pass
// (reference: encode_packed_verify_layer_major_inner, crates/qwen-llm/src/metal_dflash.rs:9045-10719;
// restore: :15649-15905; oracle: Forward::single_token_capture_layers, forward.rs:173-220).
#include <cstring>

#include "model.cuh"

namespace dfl {

dfl_status launch_group(cudaStream_t st, const MatGroup& g, const uint8_t* acts, float* part, const GemmEpilogue& ep, int* err) {
    for (size_t i = 0; i < g.mats.size(); ++i)
        DFL_CHECK(launch_gemm_fewrow(st, g.mats[i], acts, part + g.col_off[i], g.splits, ep, err, pdl_enabled(), g.total_cols));
    return DFL_OK;
}

// A group of one K-quant matrix on the tensor-memory kernel can run the glue step that follows it inside the GEMM.
static uint64_t tensor_elems(const dfl_tensor* t) {
    uint64_t n = 1;
    for (int i = 0; i < t->n_dims; ++i) n *= t->shape[i];
    return n;
}

dfl_status build_group(int device, cudaStream_t st, const TensorMap& tm, const std::vector<std::string>& names, uint64_t n_in,
                       const std::vector<uint64_t>& n_outs, MatGroup* out, bool allow_ts, int kb_group) {
    out->n_in = n_in;
    out->total_cols = 0;
    if (allow_ts) {
        // every member must consume the same packed-activation format, else the whole group stays on mma.sync
        int fmt = -1;
        for (auto& nm : names) {
            const dfl_tensor* t = tm.find(nm);
            if (!t) continue;
            const int f = !ts_supported(t->dtype) ? -2 : (t->dtype == DFL_BF16 ? ACT_TSB : ACT_TS);
            if (f == -2 || (fmt != -1 && f != fmt)) allow_ts = false;
            fmt = f;
        }
    }
    size_t i = 0;
    while (i < names.size()) {
        const dfl_tensor* t0 = tm.find(names[i]);
        if (!t0) return fail(DFL_ERR_MISSING_TENSOR, "missing tensor " + names[i]);
        // run of same-dtype tensors -> one concatenated matrix
        size_t j = i;
        uint64_t rows = 0, bytes = 0;
        while (j < names.size()) {
            const dfl_tensor* t = tm.find(names[j]);
            if (!t) return fail(DFL_ERR_MISSING_TENSOR, "missing tensor " + names[j]);
            if (t->dtype != t0->dtype || t->on_device != t0->on_device) break;
            if (kb_group > 0 && names.size() != 1) return fail(DFL_ERR_BAD_ARG, "build_group: an expert-grouped matrix stands alone");
            if (t->n_dims < 2 || (kb_group == 0 && t->shape[0] != n_in) || tensor_elems(t) != n_in * n_outs[j])
                return fail(DFL_ERR_BAD_SHAPE, "tensor " + names[j] + " has unexpected shape");
            const uint64_t want = n_outs[j] * (n_in / 256) * (uint64_t)ggml_bytes_per_256(t->dtype);
            if (n_in % 256 || ggml_bytes_per_256(t->dtype) == 0 || t->n_bytes != want)
                return fail(DFL_ERR_BAD_SHAPE, "tensor " + names[j] + ": byte count does not match dtype/shape (n_in must be a multiple of 256)");
            rows += n_outs[j];
            bytes += t->n_bytes;
            ++j;
        }
        QMatrix qm;
        if (j - i == 1) {
            DFL_CHECK(qmatrix_create(device, t0->dtype, n_in, rows, t0->data, t0->n_bytes, t0->on_device != 0, st, &qm, allow_ts, kb_group));
        } else {
            uint8_t* cat = nullptr;
            DFL_CUDA(cudaMalloc(&cat, bytes));
            uint64_t off = 0;
            for (size_t k = i; k < j; ++k) {
                const dfl_tensor* t = tm.find(names[k]);
                cudaMemcpyAsync(cat + off, t->data, t->n_bytes, t->on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, st);
                off += t->n_bytes;
            }
            dfl_status s = qmatrix_create(device, t0->dtype, n_in, rows, cat, bytes, true, st, &qm, allow_ts);
            cudaStreamSynchronize(st);
            cudaFree(cat);
            DFL_CHECK(s);
        }
        out->mats.push_back(qm);
        out->col_off.push_back(out->total_cols);
        out->total_cols += (uint32_t)rows;
        i = j;
    }
    // one split count for the whole group so that every partial slice is fully written
    QMatrix whole;
    whole.row_tiles = 0;
    whole.dtype = out->mats[0].dtype;
    whole.layout = out->mats[0].layout;
    for (auto& m : out->mats) {
        whole.row_tiles += m.row_tiles;
        if (gemm_max_kblocks_per_cta(m.dtype) < gemm_max_kblocks_per_cta(whole.dtype)) whole.dtype = m.dtype;
    }
    whole.kblocks = (int)(n_in / 256);
    if (whole.layout == LAYOUT_TS) {
        std::vector<int> tiles;
        for (auto& m : out->mats) tiles.push_back(m.row_tiles);
        out->splits = whole.dtype == DFL_BF16 ? gemm_tsb_choose_splits_multi(tiles.data(), (int)tiles.size(), whole.kblocks)
                                              : gemm_ts_choose_splits_multi(tiles.data(), (int)tiles.size(), whole.kblocks);
    } else {
        out->splits = gemm_choose_splits(whole);
    }
    return DFL_OK;
}

__global__ void decode_small_kernel(int dtype, const uint8_t* __restrict__ src, uint64_t n, float* __restrict__ out) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    if (dtype == DFL_F32) out[i] = reinterpret_cast<const float*>(src)[i];
    else if (dtype == DFL_F16) out[i] = __half2float(reinterpret_cast<const __half*>(src)[i]);
    else out[i] = __uint_as_float((uint32_t)reinterpret_cast<const uint16_t*>(src)[i] << 16);
}

dfl_status upload_f32(int device, cudaStream_t st, const TensorMap& tm, const std::string& name, uint64_t n_expected, float** out) {
    const dfl_tensor* t = tm.find(name);
    if (!t) return fail(DFL_ERR_MISSING_TENSOR, "missing tensor " + name);
    const uint64_t n = tensor_elems(t);
    if (n != n_expected) return fail(DFL_ERR_BAD_SHAPE, "tensor " + name + " has unexpected element count");
    if (t->dtype != DFL_F32 && t->dtype != DFL_F16 && t->dtype != DFL_BF16)
        return fail(DFL_ERR_UNSUPPORTED, "tensor " + name + " must be f32, f16 or bf16");
    const uint64_t esz = t->dtype == DFL_F32 ? 4 : 2;
    if (t->n_bytes != n * esz) return fail(DFL_ERR_BAD_SHAPE, "tensor " + name + " byte count mismatch");
    DFL_CUDA(cudaMalloc(out, n * 4));
    if (t->dtype == DFL_F32) {
        DFL_CUDA(cudaMemcpyAsync(*out, t->data, n * 4, t->on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, st));
        DFL_CUDA(cudaStreamSynchronize(st));
    } else {
        uint8_t* tmp = nullptr;
        DFL_CUDA(cudaMalloc(&tmp, t->n_bytes));
        cudaMemcpyAsync(tmp, t->data, t->n_bytes, t->on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, st);
        decode_small_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(t->dtype, tmp, n, *out);
        count_launch();
        cudaStreamSynchronize(st);
        cudaFree(tmp);
    }
    return DFL_OK;
}

dfl_status session_guard(const dfl_model* m, dfl_session* s, const char* what) {
    if (!m || !s) return fail(DFL_ERR_BAD_ARG, std::string(what) + ": null handle");
    if (s->m != m) return fail(DFL_ERR_BAD_ARG, std::string(what) + ": session belongs to another model");
    if (s->poisoned) return fail(DFL_ERR_POISONED, std::string(what) + ": session is poisoned by an earlier failure");
    if (m->ep_dead.load()) return fail(DFL_ERR_COLLECTIVE, std::string(what) + ": the model's expert-parallel communicator was aborted by the watchdog");
    return use_device(m->device);
}

static bool layer_is_attn(const dfl_arch& a, uint32_t il) {
    const uint32_t iv = a.full_attention_interval ? a.full_attention_interval : 1;
    return il % iv == iv - 1;
}

// Waits for everything queued on the session's stream.  A pass with collectives in it (expert-parallel model) is
// waited for under the host watchdog, not in a blocking synchronize.
dfl_status session_drain(dfl_session* s) {
    if (s->m->ep_world > 1) {
        bool aborted = false;
        dfl_status w = ep_watch_stream(s->m->ep_comm, s->st, s->ev_watch, s->m->ep_abort_host, &aborted);
        if (aborted) s->m->ep_dead.store(true);
        if (w != DFL_OK) { s->poisoned = true; return w; }
        return DFL_OK;
    }
    DFL_CUDA(cudaStreamSynchronize(s->st));
    return DFL_OK;
}

// After the stream has drained: completion check (metal/completion.rs:18) incl. the injected failure.
static dfl_status completion_check(dfl_session* s) {
    if (s->fail_next) {
        s->fail_next = false;
        s->poisoned = true;
        return fail(DFL_ERR_CUDA, "completion check failed (injected): command discarded; session poisoned");
    }
    DFL_CHECK(session_drain(s));
    dfl_status st = check_dev_err(s->st, s->err);
    if (st != DFL_OK) {
        s->poisoned = true;
        if (s->m->ep_world > 1) s->m->ep_dead.store(true);   // the ranks are no longer in step: no further pass on this model
    }
    return st;
}

dfl_status verify_core(const dfl_model* m, dfl_session* s, dfl_scratch* sc, const uint32_t* layer_ids, uint32_t n_ids,
                       const int32_t* tokens, uint32_t n, uint32_t start, bool want_head) {
    const dfl_arch& a = m->arch;
    cudaStream_t st = s->st;
    // DFL_SIDE_STREAM=0 keeps every launch of the pass on one stream
    static const bool side_enabled = [] { const char* e = getenv("DFL_SIDE_STREAM"); return !(e && e[0] == '0'); }();
    cudaStream_t side = side_enabled ? s->st_side : st, side2 = side_enabled ? s->st_side2 : st;
    auto fork_side = [&]() -> dfl_status {   // both side streams continue from here
        if (side == st) return DFL_OK;
        DFL_CUDA(cudaEventRecord(s->ev_fork, st));
        DFL_CUDA(cudaStreamWaitEvent(side, s->ev_fork, 0));
        DFL_CUDA(cudaStreamWaitEvent(side2, s->ev_fork, 0));
        return DFL_OK;
    };
    auto join_side = [&]() -> dfl_status {   // the main stream waits for what the first side stream was given
        if (side == st) return DFL_OK;
        DFL_CUDA(cudaEventRecord(s->ev_join, side));
        DFL_CUDA(cudaStreamWaitEvent(st, s->ev_join, 0));
        return DFL_OK;
    };
    auto join_side2 = [&]() -> dfl_status {   // ... and for the second
        if (side2 == st) return DFL_OK;
        DFL_CUDA(cudaEventRecord(s->ev_join2, side2));
        DFL_CUDA(cudaStreamWaitEvent(st, s->ev_join2, 0));
        return DFL_OK;
    };
    const uint64_t H = a.hidden_size, F = a.intermediate_size;
    // DFL_MOE_ALL_EXPERTS=1 streams every expert of a routed layer instead of the chosen ones
    static const bool moe_chosen_only = getenv("DFL_MOE_ALL_EXPERTS") == nullptr;
    const AttnGeom ag = m->attn_geom();
    const GdnGeom gg = m->gdn_geom();
    const int kb_h = (int)(H / GLUE_COLS);
    GemmEpilogue ep_norm;
    ep_norm.sumsq = sc->sumsq;
    ep_norm.n_sumsq = kb_h;
    ep_norm.norm_k = (float)H;
    ep_norm.eps = 1e-6f;

    memcpy(sc->pinned_i, tokens, n * sizeof(int32_t));
    DFL_CUDA(cudaMemcpyAsync(sc->tokens_dev, sc->pinned_i, n * sizeof(int32_t), cudaMemcpyHostToDevice, st));
    DFL_CHECK(launch_embed_rows(st, m->embd_dtype, m->embd_ggml, H, sc->tokens_dev, (int)n, sc->x, (int)H));

    auto norm_glue = [&](const float* part, int splits, int ld_part, const float* norm_w, bool want_xn, float* capture,
                         const int32_t* splits_dev = nullptr) -> dfl_status {
        GlueParams p;
        p.mode = GLUE_RESID;
        p.part = part; p.splits = splits; p.splits_dev = splits_dev; p.ld_part = ld_part;
        p.x = sc->x; p.ld_x = (int)H;
        p.mul_w = norm_w;
        p.acts = sc->acts_h; p.bf3 = m->act_layout;
        if (want_xn) { p.xn = sc->xn; p.ld_xn = (int)H; }
        p.sumsq = sc->sumsq;
        p.capture = capture; p.ld_capture = (int)(sc->k_layers * H);
        p.n_rows = (int)n; p.err = s->err;
        return launch_glue(st, p, H);
    };
    DFL_CHECK(norm_glue(nullptr, 0, 0, m->layers[0].attn_norm_w, !m->layers[0].is_attn, nullptr));

    int gi = 0, ai = 0;
    for (uint32_t il = 0; il < a.n_layer; ++il) {
        const LayerW& L = m->layers[il];
        const MatGroup* out_proj;
        if (L.is_attn) {
            DFL_CHECK(launch_group(st, L.qkv, sc->acts_h, sc->part, ep_norm, s->err));
            DFL_CHECK(launch_attn_front(st, ag, true, sc->part, L.qkv.splits, (int)L.qkv.total_cols, L.q_norm_w, L.k_norm_w, start, (int)n,
                                        s->k_cache[ai], s->v_cache[ai], s->kv_mode, sc->q_rot, sc->gate, nullptr));
            DFL_CHECK(launch_attn_verify(st, ag, sc->q_rot, sc->gate, s->k_cache[ai], s->v_cache[ai], s->kv_mode, start, (int)n,
                                         s->attn_partials, sc->acts_v, m->act_layout, nullptr, s->err, s->kv_capacity));
            out_proj = &L.wo;
            ++ai;
        } else {
            const int cd = gg.conv_dim();
            // qkv -> conv / norms on the main stream; the alpha / beta projection and the z projection (its own matrix
            // when its format differs from qkv's) each on a side stream: all three read only the layer's normalised
            // input and write disjoint outputs; the scan waits for alpha / beta, the gated norm for z
            const MatGroup& G = L.in_qkv_z;
            DFL_CHECK(fork_side());
            DFL_CHECK(launch_gemm_fewrow(st, G.mats[0], sc->acts_h, sc->part + G.col_off[0], G.splits, ep_norm, s->err, pdl_enabled(), G.total_cols));
            DFL_CHECK(launch_small_matmul(side, L.w_ab, sc->xn, (int)H, (int)n, H, 2 * gg.n_v, ep_norm, sc->ab[gi], 2 * gg.n_v));
            for (size_t i = 1; i < G.mats.size(); ++i)
                DFL_CHECK(launch_gemm_fewrow(side2, G.mats[i], sc->acts_h, sc->part + G.col_off[i], G.splits, ep_norm, s->err, pdl_enabled(), G.total_cols));
            const int cur = s->ssm_cur[gi];
            DFL_CHECK(launch_gdn_front(st, gg, sc->part, L.in_qkv_z.splits, (int)L.in_qkv_z.total_cols, (int)n, L.conv_w, s->conv[gi],
                                       sc->qkv_raw[gi], sc->q_n[gi], sc->k_n[gi], sc->v[gi], sc->conv_pre[gi]));
            DFL_CHECK(join_side());    // alpha / beta
            DFL_CHECK(join_side2());   // z
            DFL_CHECK(launch_gdn_scan(st, gg, s->ssm[cur][gi], s->ssm[cur ^ 1][gi], sc->q_n[gi], sc->k_n[gi], sc->v[gi], sc->ab[gi],
                                      L.dt_bias, L.a_log, (int)n, sc->part + cd, L.in_qkv_z.splits, (int)L.in_qkv_z.total_cols, L.ssm_norm_w,
                                      sc->acts_v, m->act_layout, s->err));
            s->ssm_cur[gi] = cur ^ 1;
            out_proj = &L.w_out;
            ++gi;
        }
        const bool moe = a.expert_count > 0;
        DFL_CHECK(launch_group(st, *out_proj, sc->acts_v, sc->part, GemmEpilogue{}, s->err));
        DFL_CHECK(norm_glue(sc->part, out_proj->splits, (int)out_proj->total_cols, L.post_norm_w, moe, nullptr));
        int down_splits;
        const int32_t* down_splits_dev = nullptr;
        const float* moe_part = sc->part;
        if (moe) {
            // routed experts + shared expert (forward.rs:749-824): route, then every expert of the layer as two large
            // few-row GEMMs; the glue zeroes the inner columns of the experts a token did not choose
            const int E = (int)a.expert_count, Fe = (int)a.expert_feed_forward_length, Fs = (int)m->ep_fs, En = (int)m->ep_n;
            const int inner = En * Fe + Fs;
            // Only the experts some row chose (and the shared expert) are streamed when the four gate / up blocks sit in
            // one tensor-memory matrix: router -> selection + lists -> GEMM over the listed tiles, one after the other.
            // Otherwise every expert is streamed and the router and the selection run beside that GEMM.
            const MatGroup& GU = L.moe_gate_up;
            const bool down_chosen = L.moe_down.mats.size() == 1 && L.moe_down.mats[0].layout == LAYOUT_TS && Fe % TILE_K == 0;
            const bool chosen_only = moe_chosen_only && GU.mats.size() == 1 && GU.mats[0].layout == LAYOUT_TS && Fe % TILE_R == 0 && Fs % TILE_R == 0;
            if (chosen_only) {
                const int min_tiles = gemm_ts_ctas_per_split(GU.mats[0].row_tiles, GU.splits);
                const int down_tiles = down_chosen ? L.moe_down.mats[0].row_tiles : 1, down_max = down_chosen ? L.moe_down.splits : 0;
                int32_t* kb_map = down_chosen ? sc->moe_kb_map : nullptr;
                DFL_CHECK(launch_small_matmul(st, L.router_w, sc->xn, (int)H, (int)n, H, E + 1, ep_norm, sc->route_logits, E + 1));
                if (moe_route_lists_fused(E)) {
                    DFL_CHECK(launch_moe_route_lists(st, sc->route_logits, E + 1, E, (int)a.expert_used_count, (int)n, sc->route_w, sc->route_sg,
                                                     sc->route_idx, (int)m->ep_e0, En, Fe / TILE_R, Fs / TILE_R, min_tiles, sc->moe_tile_map,
                                                     sc->moe_n_tiles, Fe / TILE_K, 1, kb_map, sc->moe_n_tiles + 1, gemm_ts_kc(), down_tiles, down_max, s->err));
                } else {
                    DFL_CHECK(launch_moe_route(st, sc->route_logits, E + 1, E, (int)a.expert_used_count, (int)n, sc->route_w, sc->route_sg, sc->route_idx, s->err));
                    DFL_CHECK(launch_moe_tiles(st, sc->route_w, (int)n, E, (int)m->ep_e0, En, Fe / TILE_R, Fs / TILE_R, min_tiles, sc->moe_tile_map,
                                               sc->moe_n_tiles, Fe / TILE_K, 1, kb_map, sc->moe_n_tiles + 1, gemm_ts_kc(), down_tiles, down_max));
                }
                GemmEpilogue ep_gu = ep_norm;
                ep_gu.tile_map = sc->moe_tile_map;
                ep_gu.n_tiles = sc->moe_n_tiles;
                DFL_CHECK(launch_group(st, GU, sc->acts_h, sc->part, ep_gu, s->err));
            } else {
                DFL_CHECK(fork_side());
                DFL_CHECK(launch_small_matmul(side, L.router_w, sc->xn, (int)H, (int)n, H, E + 1, ep_norm, sc->route_logits, E + 1));
                DFL_CHECK(launch_moe_route(side, sc->route_logits, E + 1, E, (int)a.expert_used_count, (int)n, sc->route_w, sc->route_sg, sc->route_idx, s->err));
                DFL_CHECK(launch_group(st, GU, sc->acts_h, sc->part, ep_norm, s->err));
                DFL_CHECK(join_side());
            }
            GlueParams p;
            p.mode = GLUE_SWIGLU;
            p.part = sc->part; p.splits = L.moe_gate_up.splits; p.ld_part = (int)L.moe_gate_up.total_cols;
            p.swiglu_f = inner;
            p.route_w = sc->route_w; p.route_sg = sc->route_sg; p.route_e = E; p.route_f = Fe;
            p.route_e0 = (int)m->ep_e0; p.route_n = En;
            p.pre_scale = 1.0f / 64.0f;
            p.acts = sc->acts_f; p.bf3 = m->act_layout;
            p.n_rows = (int)n; p.err = s->err;
            DFL_CHECK(launch_glue(st, p, (uint64_t)inner));
            GemmEpilogue ep_down;
            ep_down.out_scale = 64.0f;
            // partial slices: the shared expert's first, then the routed experts' - as many as the split count in use,
            // which follows the number of chosen experts (written beside the lists) when only those are summed over
            GemmEpilogue ep_down_exps = ep_down;
            const int sh_splits = Fs > 0 ? L.moe_down_sh.splits : 0;
            if (chosen_only && down_chosen) {
                ep_down_exps.kb_map = sc->moe_kb_map;
                ep_down_exps.n_kb = sc->moe_n_tiles + 1;
                ep_down_exps.dynamic_splits = true;
                down_splits_dev = sc->moe_n_tiles + 2;
            }
            // the shared expert's small down projection runs beside the routed experts' on the side stream
            if (Fs > 0) {
                DFL_CHECK(fork_side());
                DFL_CHECK(launch_group(side, L.moe_down_sh, sc->acts_f + (uint64_t)(En * Fe / TILE_K) * act_chunk_bytes(m->act_layout), sc->part,
                                       ep_down, s->err));
            }
            DFL_CHECK(launch_group(st, L.moe_down, sc->acts_f, sc->part + (uint64_t)sh_splits * MAX_ROWS * H, ep_down_exps, s->err));
            if (Fs > 0) DFL_CHECK(join_side());
            down_splits = sh_splits + (down_splits_dev ? 0 : L.moe_down.splits);
            if (m->ep_world > 1 && m->ep_p2p) {
                // this rank's slices summed and pushed into every rank's receive buffer; the glue below adds the ranks'
                // slots in rank order, so every rank continues with the same [16][H] block output
                const uint32_t seq = ++m->ep_seq;
                DFL_CHECK(launch_ep_push_sum(st, sc->part, down_splits, down_splits_dev, H, m->ep_peers, m->ep_rank, m->ep_world, seq, m->ep_abort_dev, s->err));
                down_splits_dev = nullptr;
                moe_part = m->ep_peers.base[m->ep_rank] + (uint64_t)(seq & 1u) * m->ep_world * MAX_ROWS * H;
                down_splits = m->ep_world;
            } else if (m->ep_world > 1) {
                // the same through the library: local sum, then an all-reduce over the ranks
                DFL_CHECK(launch_reduce_partials(st, sc->part, down_splits, MAX_ROWS, H, sc->moe_out, (int)H, down_splits_dev));
                down_splits_dev = nullptr;
                DFL_CHECK(ep_all_reduce_sum(m->ep_comm, sc->moe_out, (size_t)MAX_ROWS * H, st));
                moe_part = sc->moe_out;
                down_splits = 1;
            }
        } else {
        // dense SwiGLU FFN (forward.rs:725-747)
        {
            GlueParams p;
            p.mode = GLUE_SWIGLU;
            p.part = sc->part; p.splits = L.gate_up.splits; p.ld_part = (int)L.gate_up.total_cols;
            p.swiglu_f = (int)F;
            p.pre_scale = 1.0f / 64.0f;  // keeps silu(g)*u inside the f16 operand range; undone in the GEMM epilogue
            p.acts = sc->acts_f; p.bf3 = m->act_layout;
            p.n_rows = (int)n; p.err = s->err;
            DFL_CHECK(launch_group(st, L.gate_up, sc->acts_h, sc->part, ep_norm, s->err));
            DFL_CHECK(launch_glue(st, p, F));
        }
        down_splits = L.down.splits;
        }
        float* cap = nullptr;
        for (uint32_t k = 0; k < n_ids; ++k)
            if (layer_ids[k] == il) { cap = sc->capture + (uint64_t)k * H; break; }   // the kernel fills the first slot of this layer
        const bool last = il + 1 == a.n_layer;
        const float* next_w = last ? m->out_norm_w : m->layers[il + 1].attn_norm_w;
        const bool next_gdn = !last && !m->layers[il + 1].is_attn;
        if (!moe) {
            GemmEpilogue ep_down;
            ep_down.out_scale = 64.0f;
            DFL_CHECK(launch_group(st, L.down, sc->acts_f, sc->part, ep_down, s->err));
        }
        DFL_CHECK(norm_glue(moe_part, down_splits, (int)H, next_w, next_gdn, cap, down_splits_dev));
        if (cap) {
            // duplicate slots (same layer listed twice) get a device copy of the first one
            bool first = true;
            for (uint32_t k = 0; k < n_ids; ++k) {
                if (layer_ids[k] != il) continue;
                if (first) { first = false; continue; }
                DFL_CUDA(cudaMemcpy2DAsync(sc->capture + (uint64_t)k * H, sc->k_layers * H * 4, cap, sc->k_layers * H * 4, H * 4, n,
                                           cudaMemcpyDeviceToDevice, st));
            }
        }
    }
    if (want_head) {
        const uint64_t V = a.vocab_size;
        const MatGroup& lm = m->lm_head;
        float* logits = sc->logits;
        if (lm.splits == 1) {
            DFL_CHECK(launch_group(st, lm, sc->acts_h, logits, ep_norm, s->err));
            DFL_CHECK(launch_argmax_top2(st, logits, (int)n, V, V, sc->argmax, sc->gap, sc->am_scratch));
        } else {
            DFL_CHECK(launch_group(st, lm, sc->acts_h, sc->part, ep_norm, s->err));
            DFL_CHECK(launch_reduce_argmax_top2(st, sc->part, lm.splits, (int)n, V, logits, V, sc->argmax, sc->gap, sc->am_scratch));
        }
    }
    DFL_CHECK(join_side());   // whatever the side streams still hold belongs to this pass
    DFL_CHECK(join_side2());
    s->kv_n_pos = start + n;
    sc->last_n = n;
    sc->last_n_verify = n;
    sc->last_start = start;
    sc->have_block = true;
    return DFL_OK;
}

}  // namespace dfl

using namespace dfl;

extern "C" {

}  // extern "C"

static dfl_status model_create_impl(int32_t device, const dfl_arch* arch, const dfl_tensor* tensors, uint64_t n_tensors, int ep_rank,
                                    int ep_world, const uint8_t* nccl_id, dfl_model** out) {
    if (!arch || !tensors || !out) return fail(DFL_ERR_BAD_ARG, "model_create: null argument");
    *out = nullptr;
    if (ep_world < 1 || ep_rank < 0 || ep_rank >= ep_world) return fail(DFL_ERR_BAD_ARG, "model_create: expert-parallel rank / world");
    if (ep_world > 1 && (arch->expert_count == 0 || arch->expert_count % ep_world || !nccl_id))
        return fail(DFL_ERR_BAD_ARG, "model_create: expert parallelism needs a routed-expert model whose expert count divides by the world size");
    DFL_CHECK(use_device(device));
    const dfl_arch& a = *arch;
    if (a.n_layer == 0 || a.hidden_size % 256 || a.hidden_size == 0) return fail(DFL_ERR_BAD_SHAPE, "model_create: hidden size must be a positive multiple of 256");
    if (a.expert_count > 0 && (a.expert_feed_forward_length == 0 || a.expert_feed_forward_length % 256 || a.expert_shared_feed_forward_length == 0 ||
                               a.expert_shared_feed_forward_length % 256 || a.expert_used_count == 0 || a.expert_used_count > a.expert_count))
        return fail(DFL_ERR_BAD_SHAPE, "model_create: expert FFN widths must be positive multiples of 256 and 1 <= used <= count");
    if (a.intermediate_size % 256) return fail(DFL_ERR_BAD_SHAPE, "model_create: FFN width must be a multiple of 256");
    if (a.gdn_head_dim != 128 || a.gdn_conv_kernel != 4) return fail(DFL_ERR_UNSUPPORTED, "model_create: GDN head_dim must be 128 and conv kernel 4");
    if (a.attn_head_dim != 128 && a.attn_head_dim != 256) return fail(DFL_ERR_UNSUPPORTED, "model_create: attention head_dim must be 128 or 256");
    if (a.n_kv_heads == 0 || a.n_q_heads % a.n_kv_heads || a.gdn_n_k_heads == 0 || a.gdn_n_v_heads % a.gdn_n_k_heads)
        return fail(DFL_ERR_BAD_SHAPE, "model_create: head counts");
    if (((uint64_t)a.n_q_heads * a.attn_head_dim) % 256 || ((uint64_t)a.gdn_n_v_heads * 128) % 256)
        return fail(DFL_ERR_BAD_SHAPE, "model_create: projection widths must be multiples of 256");
    TensorMap tm;
    for (uint64_t i = 0; i < n_tensors; ++i) {
        if (!tensors[i].name || !tensors[i].data) return fail(DFL_ERR_BAD_ARG, "model_create: tensor without name or data");
        tm.t[tensors[i].name] = &tensors[i];
    }
    auto* m = new dfl_model();
    m->device = device;
    m->ep_rank = ep_rank;
    m->ep_world = ep_world;
    m->ep_n = arch->expert_count / (uint32_t)ep_world;
    m->ep_e0 = (uint32_t)ep_rank * m->ep_n;
    m->ep_fs = ep_rank == 0 ? arch->expert_shared_feed_forward_length : 0;
    std::vector<dfl_tensor> sliced;   // this rank's views of the stacked expert tensors
    sliced.reserve(3 * (size_t)arch->n_layer);
    // One kernel family per model, so that every packed-activation buffer has a single format: the tensor-memory GEMM
    // when every 2-D quantised tensor has a row-lane layout (Q4_K / Q5_K / Q6_K), else - a model that holds Q8_0
    // matrices - the mma.sync kernel for all of them.
    bool allow_ts = true;
    for (uint64_t i = 0; i < n_tensors; ++i)
        if (tensors[i].n_dims >= 2 && stage_bytes_of(tensors[i].dtype) != 0 &&
            !(tensors[i].dtype == DFL_Q4_K || tensors[i].dtype == DFL_Q5_K || tensors[i].dtype == DFL_Q6_K))
            allow_ts = false;
    m->act_layout = allow_ts ? ACT_TS : ACT_F16;
    m->arch = a;
    cudaStream_t st = 0;
    const uint64_t H = a.hidden_size, F = a.intermediate_size, V = a.vocab_size;
    const uint64_t hd = a.attn_head_dim, q_dim = a.n_q_heads * hd, kv_dim = a.n_kv_heads * hd;
    const uint64_t conv_dim = (2ull * a.gdn_n_k_heads + a.gdn_n_v_heads) * 128, v_dim = a.gdn_n_v_heads * 128ull;
    dfl_status s = DFL_OK;
    auto blk = [](uint32_t il, const char* suffix) { return "blk." + std::to_string(il) + "." + suffix; };
#define MC(expr)                      \
    do {                              \
        s = (expr);                   \
        if (s != DFL_OK) goto failed; \
    } while (0)
    {
        const dfl_tensor* te = tm.find("token_embd.weight");
        if (!te) { s = fail(DFL_ERR_MISSING_TENSOR, "missing tensor token_embd.weight"); goto failed; }
        const uint64_t want = V * (H / 256) * (uint64_t)ggml_bytes_per_256(te->dtype);
        if (ggml_bytes_per_256(te->dtype) == 0 || te->n_bytes != want) { s = fail(DFL_ERR_BAD_SHAPE, "token_embd.weight: byte count"); goto failed; }
        if (cudaMalloc(&m->embd_ggml, te->n_bytes) != cudaSuccess) { s = fail(DFL_ERR_OOM, "token_embd"); goto failed; }
        cudaMemcpy(m->embd_ggml, te->data, te->n_bytes, te->on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice);
        m->embd_dtype = te->dtype;
        const char* head_name = tm.find("output.weight") ? "output.weight" : "token_embd.weight";  // tied embeddings, loader.rs:445
        MC(build_group(device, st, tm, {head_name}, H, {V}, &m->lm_head, allow_ts));
        MC(upload_f32(device, st, tm, "output_norm.weight", H, &m->out_norm_w));
        m->verify_weight_bytes = m->lm_head.ggml_bytes();
        m->verify_resident_bytes = m->lm_head.bytes();
    }
    m->layers.resize(a.n_layer);
    for (uint32_t il = 0; il < a.n_layer; ++il) {
        LayerW& L = m->layers[il];
        L.is_attn = layer_is_attn(a, il);
        MC(upload_f32(device, st, tm, blk(il, "attn_norm.weight"), H, &L.attn_norm_w));
        MC(upload_f32(device, st, tm, blk(il, "post_attention_norm.weight"), H, &L.post_norm_w));
        if (L.is_attn) {
            ++m->n_attn;
            MC(build_group(device, st, tm, {blk(il, "attn_q.weight"), blk(il, "attn_k.weight"), blk(il, "attn_v.weight")}, H,
                           {2 * q_dim, kv_dim, kv_dim}, &L.qkv, allow_ts));
            MC(build_group(device, st, tm, {blk(il, "attn_output.weight")}, q_dim, {H}, &L.wo, allow_ts));
            MC(upload_f32(device, st, tm, blk(il, "attn_q_norm.weight"), hd, &L.q_norm_w));
            MC(upload_f32(device, st, tm, blk(il, "attn_k_norm.weight"), hd, &L.k_norm_w));
            m->verify_weight_bytes += L.qkv.ggml_bytes() + L.wo.ggml_bytes();
            m->verify_resident_bytes += L.qkv.bytes() + L.wo.bytes();
        } else {
            ++m->n_gdn;
            MC(build_group(device, st, tm, {blk(il, "attn_qkv.weight"), blk(il, "attn_gate.weight")}, H, {conv_dim, v_dim}, &L.in_qkv_z, allow_ts));
            MC(build_group(device, st, tm, {blk(il, "ssm_out.weight")}, v_dim, {H}, &L.w_out, allow_ts));
            {
                float *al = nullptr, *be = nullptr;
                MC(upload_f32(device, st, tm, blk(il, "ssm_alpha.weight"), H * a.gdn_n_v_heads, &al));
                s = upload_f32(device, st, tm, blk(il, "ssm_beta.weight"), H * a.gdn_n_v_heads, &be);
                if (s != DFL_OK) { cudaFree(al); goto failed; }
                cudaMalloc(&L.w_ab, 2 * H * a.gdn_n_v_heads * 4);
                cudaMemcpy(L.w_ab, al, H * a.gdn_n_v_heads * 4, cudaMemcpyDeviceToDevice);
                cudaMemcpy(L.w_ab + H * a.gdn_n_v_heads, be, H * a.gdn_n_v_heads * 4, cudaMemcpyDeviceToDevice);
                cudaFree(al);
                cudaFree(be);
            }
            MC(upload_f32(device, st, tm, blk(il, "ssm_a"), a.gdn_n_v_heads, &L.a_log));
            MC(upload_f32(device, st, tm, blk(il, "ssm_dt.bias"), a.gdn_n_v_heads, &L.dt_bias));
            MC(upload_f32(device, st, tm, blk(il, "ssm_conv1d.weight"), conv_dim * 4, &L.conv_w));
            MC(upload_f32(device, st, tm, blk(il, "ssm_norm.weight"), 128, &L.ssm_norm_w));
            m->verify_weight_bytes += L.in_qkv_z.ggml_bytes() + L.w_out.ggml_bytes() + 2 * H * a.gdn_n_v_heads * 4;
            m->verify_resident_bytes += L.in_qkv_z.bytes() + L.w_out.bytes() + 2 * H * a.gdn_n_v_heads * 4;
        }
        if (a.expert_count > 0) {
            // forward.rs:749-824; tensor shapes as in loader.rs (experts stacked along the last ggml dimension)
            if (!allow_ts) { s = fail(DFL_ERR_UNSUPPORTED, "model_create: the routed-expert FFN needs Q4_K / Q5_K / Q6_K matrices"); goto failed; }
            const uint64_t E = a.expert_count, Fe = a.expert_feed_forward_length, Fs = m->ep_fs, En = m->ep_n;
            if (ep_world > 1) {
                // experts are stacked along the last ggml dimension: this rank's range is one contiguous byte range
                for (const char* nm : {"ffn_gate_exps.weight", "ffn_up_exps.weight", "ffn_down_exps.weight"}) {
                    const dfl_tensor* t = tm.find(blk(il, nm));
                    if (!t) { s = fail(DFL_ERR_MISSING_TENSOR, "missing tensor " + blk(il, nm)); goto failed; }
                    if (t->n_dims != 3 || t->shape[2] != E || t->n_bytes % E) { s = fail(DFL_ERR_BAD_SHAPE, blk(il, nm) + ": expected [.., .., n_expert]"); goto failed; }
                    dfl_tensor v = *t;
                    v.shape[2] = En;
                    v.n_bytes = t->n_bytes / E * En;
                    v.data = static_cast<const uint8_t*>(t->data) + t->n_bytes / E * m->ep_e0;
                    sliced.push_back(v);
                    tm.t[blk(il, nm)] = &sliced.back();
                }
            }
            if (Fs > 0) {
                MC(build_group(device, st, tm, {blk(il, "ffn_gate_exps.weight"), blk(il, "ffn_gate_shexp.weight"), blk(il, "ffn_up_exps.weight"),
                                               blk(il, "ffn_up_shexp.weight")}, H, {En * Fe, Fs, En * Fe, Fs}, &L.moe_gate_up, allow_ts));
                MC(build_group(device, st, tm, {blk(il, "ffn_down_shexp.weight")}, Fs, {H}, &L.moe_down_sh, allow_ts));
            } else {
                MC(build_group(device, st, tm, {blk(il, "ffn_gate_exps.weight"), blk(il, "ffn_up_exps.weight")}, H, {En * Fe, En * Fe},
                               &L.moe_gate_up, allow_ts));
            }
            MC(build_group(device, st, tm, {blk(il, "ffn_down_exps.weight")}, En * Fe, {H}, &L.moe_down, allow_ts, (int)(Fe / 256)));
            {
                float *rw = nullptr, *sgw = nullptr;
                MC(upload_f32(device, st, tm, blk(il, "ffn_gate_inp.weight"), H * E, &rw));
                s = upload_f32(device, st, tm, blk(il, "ffn_gate_inp_shexp.weight"), H, &sgw);
                if (s != DFL_OK) { cudaFree(rw); goto failed; }
                cudaMalloc(&L.router_w, (E + 1) * H * 4);
                cudaMemcpy(L.router_w, rw, E * H * 4, cudaMemcpyDeviceToDevice);
                cudaMemcpy(L.router_w + E * H, sgw, H * 4, cudaMemcpyDeviceToDevice);
                cudaFree(rw);
                cudaFree(sgw);
            }
            m->verify_weight_bytes += L.moe_gate_up.ggml_bytes() + L.moe_down.ggml_bytes() + L.moe_down_sh.ggml_bytes() + (E + 1) * H * 4;
            m->verify_resident_bytes += L.moe_gate_up.bytes() + L.moe_down.bytes() + L.moe_down_sh.bytes() + (E + 1) * H * 4;
        } else {
            MC(build_group(device, st, tm, {blk(il, "ffn_gate.weight"), blk(il, "ffn_up.weight")}, H, {F, F}, &L.gate_up, allow_ts));
            MC(build_group(device, st, tm, {blk(il, "ffn_down.weight")}, F, {H}, &L.down, allow_ts));
            m->verify_weight_bytes += L.gate_up.ggml_bytes() + L.down.ggml_bytes();
            m->verify_resident_bytes += L.gate_up.bytes() + L.down.bytes();
        }
    }
#undef MC
    cudaDeviceSynchronize();
    if (ep_world > 1) {
        s = ep_comm_create(ep_rank, ep_world, nccl_id, &m->ep_comm);
        if (s != DFL_OK) goto failed;
        // DFL_EP_COMBINE=nccl keeps the block-output sum on ncclAllReduce (for comparison); the default is the
        // peer-memory combine of ep_combine.cu
        const char* e = getenv("DFL_EP_COMBINE");
        if (!(e && e[0] == 'n') && ep_world <= EP_MAX_WORLD) {
            const uint64_t recv_bytes = ep_recv_floats(ep_world, H) * 4;
            const uint64_t flag_bytes = 2ull * ep_world * ep_combine_ctas(H) * 4;
            void* local = nullptr;
            if (cudaMalloc(&local, recv_bytes + flag_bytes) != cudaSuccess) { s = fail(DFL_ERR_OOM, "model_create: exchange buffer"); goto failed; }
            cudaMemset(local, 0, recv_bytes + flag_bytes);
            cudaDeviceSynchronize();
            void* peers[EP_MAX_WORLD] = {};
            s = ep_p2p_exchange(m->ep_comm, ep_rank, ep_world, local, st, peers);
            if (s != DFL_OK) { cudaFree(local); goto failed; }
            for (int p = 0; p < ep_world; ++p) m->ep_peers.base[p] = (float*)peers[p];
            m->ep_peers.flags_off = recv_bytes;
            if (cudaHostAlloc((void**)&m->ep_abort_host, sizeof(int), cudaHostAllocMapped) != cudaSuccess ||
                cudaHostGetDevicePointer((void**)&m->ep_abort_dev, m->ep_abort_host, 0) != cudaSuccess) {
                s = fail(DFL_ERR_OOM, "model_create: abort word");
                m->ep_p2p = true;   // so that the destructor unmaps what was mapped
                goto failed;
            }
            *m->ep_abort_host = 0;
            m->ep_p2p = true;
        }
    }
    *out = m;
    return DFL_OK;
failed:
    dfl_model_destroy(m);
    return s;
}

extern "C" {

dfl_status dfl_model_create(int32_t device, const dfl_arch* arch, const dfl_tensor* tensors, uint64_t n_tensors, dfl_model** out) {
    return model_create_impl(device, arch, tensors, n_tensors, 0, 1, nullptr, out);
}
dfl_status dfl_ep_unique_id(uint8_t* id_out) {
    if (!id_out) return fail(DFL_ERR_BAD_ARG, "ep_unique_id: null argument");
    return ep_unique_id(id_out);
}
dfl_status dfl_model_create_ep(int32_t device, const dfl_arch* arch, const dfl_tensor* tensors, uint64_t n_tensors, int32_t ep_rank,
                               int32_t ep_world, const uint8_t* nccl_id, dfl_model** out) {
    return model_create_impl(device, arch, tensors, n_tensors, ep_rank, ep_world, nccl_id, out);
}

void dfl_model_destroy(dfl_model* m) {
    if (!m) return;
    cudaSetDevice(m->device);
    for (auto& L : m->layers) {
        L.qkv.release(); L.wo.release(); L.in_qkv_z.release(); L.w_out.release(); L.gate_up.release(); L.down.release();
        L.moe_gate_up.release(); L.moe_down.release(); L.moe_down_sh.release();
        cudaFree(L.router_w);
        for (float* p : {L.attn_norm_w, L.post_norm_w, L.q_norm_w, L.k_norm_w, L.w_ab, L.a_log, L.dt_bias, L.conv_w, L.ssm_norm_w})
            if (p) cudaFree(p);
    }
    m->lm_head.release();
    if (m->ep_p2p) {
        // Peers unmap first; a rank frees its buffer only once every rank has unmapped it, which a bounded barrier
        // establishes.  When the peers do not answer within two seconds (they have gone, or never destroy their
        // model) the communicator is aborted and the buffer stays allocated until the process ends.
        void* peers[EP_MAX_WORLD];
        for (int p = 0; p < EP_MAX_WORLD; ++p) peers[p] = m->ep_peers.base[p];
        ep_p2p_close(m->ep_rank, m->ep_world, peers);
        if (!m->ep_dead.load() && m->ep_comm) {
            if (ep_barrier_bounded(m->ep_comm, 0, 2000)) cudaFree(m->ep_peers.base[m->ep_rank]);
            else m->ep_dead.store(true);
        }
        if (m->ep_abort_host) cudaFreeHost(m->ep_abort_host);
    }
    ep_comm_destroy(m->ep_comm, m->ep_dead.load());
    if (m->embd_ggml) cudaFree(m->embd_ggml);
    if (m->out_norm_w) cudaFree(m->out_norm_w);
    delete m;
}

uint64_t dfl_model_verify_weight_bytes(const dfl_model* m) { return m ? m->verify_weight_bytes : 0; }
uint64_t dfl_model_verify_resident_bytes(const dfl_model* m) { return m ? m->verify_resident_bytes : 0; }

dfl_status dfl_session_create(const dfl_model* m, uint32_t kv_capacity, int32_t kv_f16, dfl_session** out) {
    if (!m || !out) return fail(DFL_ERR_BAD_ARG, "session_create: null argument");
    *out = nullptr;
    if (kv_capacity == 0) return fail(DFL_ERR_BAD_ARG, "session_create: kv_capacity must be positive");
    DFL_CHECK(use_device(m->device));
    auto* s = new dfl_session();
    s->m = m;
    s->kv_capacity = kv_capacity;
    s->kv_f16 = kv_f16 != 0;
    const dfl_arch& a = m->arch;
    // Tiled storage (the tcgen05 attention kernel) where the KV scan is what a verify pass spends its time on: fp16
    // caches of 16384 positions and more, when the geometry fits.  DFL_ATTN_TILED=1 / 0 forces it on (where supported)
    // or off.
    s->kv_mode = s->kv_f16 ? KV_F16_ROWS : KV_F32_ROWS;
    if (m->n_attn && attn_t5_supported(m->attn_geom(), s->kv_f16)) {
        const char* e = getenv("DFL_ATTN_TILED");
        if (e ? e[0] == '1' : kv_capacity >= 16384) s->kv_mode = KV_F16_TILED;
    }
    const size_t cap_alloc = s->kv_mode == KV_F16_TILED ? ((size_t)kv_capacity + KV_TILE_KEYS - 1) / KV_TILE_KEYS * KV_TILE_KEYS : kv_capacity;
    const size_t kv_elems = cap_alloc * a.n_kv_heads * a.attn_head_dim;
    const size_t kv_bytes = kv_elems * (s->kv_f16 ? 2 : 4);
    const size_t conv_bytes = (size_t)3 * m->gdn_geom().conv_dim() * 4;
    const size_t ssm_bytes = (size_t)a.gdn_n_v_heads * 128 * 128 * 4;
    bool ok = cudaStreamCreateWithFlags(&s->st, cudaStreamNonBlocking) == cudaSuccess;
    for (int i = 0; i < m->n_attn && ok; ++i) {
        void *k = nullptr, *v = nullptr;
        ok = cudaMalloc(&k, kv_bytes) == cudaSuccess && cudaMalloc(&v, kv_bytes) == cudaSuccess;
        // whole tiles go through the tensor cores, positions not yet written included: they must hold finite values
        if (ok && s->kv_mode == KV_F16_TILED) { cudaMemset(k, 0, kv_bytes); cudaMemset(v, 0, kv_bytes); }
        s->k_cache.push_back(k);
        s->v_cache.push_back(v);
    }
    for (int i = 0; i < m->n_gdn && ok; ++i) {
        float *c = nullptr, *s0 = nullptr, *s1 = nullptr;
        ok = cudaMalloc(&c, conv_bytes) == cudaSuccess && cudaMalloc(&s0, ssm_bytes) == cudaSuccess && cudaMalloc(&s1, ssm_bytes) == cudaSuccess;
        if (ok) { cudaMemset(c, 0, conv_bytes); cudaMemset(s0, 0, ssm_bytes); cudaMemset(s1, 0, ssm_bytes); }
        s->conv.push_back(c);
        s->ssm[0].push_back(s0);
        s->ssm[1].push_back(s1);
        s->ssm_cur.push_back(0);
    }
    if (ok && m->n_attn) ok = cudaMalloc(&s->attn_partials, attn_partials_floats(m->attn_geom(), (uint32_t)cap_alloc) * 4) == cudaSuccess;   // two records per 128-position tile in tiled storage
    ok = ok && cudaMalloc(&s->err, 4) == cudaSuccess;
    ok = ok && cudaEventCreate(&s->ev0) == cudaSuccess && cudaEventCreate(&s->ev1) == cudaSuccess;
    ok = ok && cudaStreamCreateWithFlags(&s->st_side, cudaStreamNonBlocking) == cudaSuccess &&
         cudaStreamCreateWithFlags(&s->st_side2, cudaStreamNonBlocking) == cudaSuccess;
    ok = ok && cudaEventCreateWithFlags(&s->ev_fork, cudaEventDisableTiming) == cudaSuccess &&
         cudaEventCreateWithFlags(&s->ev_join, cudaEventDisableTiming) == cudaSuccess &&
         cudaEventCreateWithFlags(&s->ev_join2, cudaEventDisableTiming) == cudaSuccess &&
         cudaEventCreateWithFlags(&s->ev_watch, cudaEventDisableTiming) == cudaSuccess;
    if (!ok) {
        std::string why = cudaGetErrorString(cudaGetLastError());
        dfl_session_destroy(s);
        return fail(DFL_ERR_OOM, "session_create: allocation failed: " + why);
    }
    cudaMemset(s->err, 0, 4);
    cudaDeviceSynchronize();
    *out = s;
    return DFL_OK;
}

void dfl_session_destroy(dfl_session* s) {
    if (!s) return;
    cudaSetDevice(s->m->device);
    for (void* p : s->k_cache) cudaFree(p);
    for (void* p : s->v_cache) cudaFree(p);
    for (float* p : s->conv) cudaFree(p);
    for (float* p : s->ssm[0]) cudaFree(p);
    for (float* p : s->ssm[1]) cudaFree(p);
    cudaFree(s->attn_partials);
    cudaFree(s->err);
    if (s->ev0) cudaEventDestroy(s->ev0);
    if (s->ev1) cudaEventDestroy(s->ev1);
    if (s->ev_fork) cudaEventDestroy(s->ev_fork);
    if (s->ev_join) cudaEventDestroy(s->ev_join);
    if (s->ev_join2) cudaEventDestroy(s->ev_join2);
    if (s->ev_watch) cudaEventDestroy(s->ev_watch);
    if (s->st_side) cudaStreamDestroy(s->st_side);
    if (s->st_side2) cudaStreamDestroy(s->st_side2);
    if (s->st) cudaStreamDestroy(s->st);
    delete s;
}

uint32_t dfl_session_kv_n_pos(const dfl_session* s) { return s ? s->kv_n_pos : 0; }
int32_t dfl_session_poisoned(const dfl_session* s) { return s && s->poisoned ? 1 : 0; }
void dfl_session_fail_next_completion(dfl_session* s) { if (s) s->fail_next = true; }

dfl_status dfl_session_read_gdn_state(const dfl_session* s, uint32_t gdn_index, float* ssm_out, uint64_t n_ssm, float* conv_out, uint64_t n_conv) {
    if (!s) return fail(DFL_ERR_BAD_ARG, "read_gdn_state: null session");
    if (gdn_index >= s->conv.size()) return fail(DFL_ERR_BAD_ARG, "read_gdn_state: layer index");
    DFL_CHECK(use_device(s->m->device));
    const uint64_t want_ssm = (uint64_t)s->m->arch.gdn_n_v_heads * 128 * 128, want_conv = 3ull * s->m->gdn_geom().conv_dim();
    DFL_CUDA(cudaStreamSynchronize(s->st));
    if (ssm_out) {
        if (n_ssm != want_ssm) return fail(DFL_ERR_BAD_SHAPE, "read_gdn_state: ssm size");
        DFL_CUDA(cudaMemcpy(ssm_out, s->ssm[s->ssm_cur[gdn_index]][gdn_index], want_ssm * 4, cudaMemcpyDeviceToHost));
    }
    if (conv_out) {
        if (n_conv != want_conv) return fail(DFL_ERR_BAD_SHAPE, "read_gdn_state: conv size");
        DFL_CUDA(cudaMemcpy(conv_out, s->conv[gdn_index], want_conv * 4, cudaMemcpyDeviceToHost));
    }
    return DFL_OK;
}

dfl_status dfl_session_read_kv(const dfl_session* s, uint32_t attn_index, uint32_t pos, float* k_out, float* v_out, uint64_t n) {
    if (!s || !k_out || !v_out) return fail(DFL_ERR_BAD_ARG, "read_kv: null argument");
    if (attn_index >= s->k_cache.size() || pos >= s->kv_n_pos) return fail(DFL_ERR_BAD_ARG, "read_kv: index");
    const uint64_t stride = (uint64_t)s->m->arch.n_kv_heads * s->m->arch.attn_head_dim;
    if (n != stride) return fail(DFL_ERR_BAD_SHAPE, "read_kv: row size");
    DFL_CHECK(use_device(s->m->device));
    DFL_CUDA(cudaStreamSynchronize(s->st));
    if (s->kv_mode == KV_F16_TILED) {
        std::vector<__half> hk(stride), hv(stride);
        __half* tmp = nullptr;
        DFL_CUDA(cudaMalloc(&tmp, 2 * stride * 2));
        dfl_status st = launch_kv_tiled_to_rows(s->st, s->k_cache[attn_index], false, (int)s->m->arch.n_kv_heads, pos, 1, tmp);
        if (st == DFL_OK) st = launch_kv_tiled_to_rows(s->st, s->v_cache[attn_index], true, (int)s->m->arch.n_kv_heads, pos, 1, tmp + stride);
        cudaError_t e = cudaStreamSynchronize(s->st);
        if (st == DFL_OK && e == cudaSuccess) {
            cudaMemcpy(hk.data(), tmp, stride * 2, cudaMemcpyDeviceToHost);
            e = cudaMemcpy(hv.data(), tmp + stride, stride * 2, cudaMemcpyDeviceToHost);
        }
        cudaFree(tmp);
        DFL_CHECK(st);
        DFL_CUDA(e);
        for (uint64_t i = 0; i < stride; ++i) { k_out[i] = __half2float(hk[i]); v_out[i] = __half2float(hv[i]); }
    } else if (s->kv_f16) {
        std::vector<__half> hk(stride), hv(stride);
        DFL_CUDA(cudaMemcpy(hk.data(), (const __half*)s->k_cache[attn_index] + pos * stride, stride * 2, cudaMemcpyDeviceToHost));
        DFL_CUDA(cudaMemcpy(hv.data(), (const __half*)s->v_cache[attn_index] + pos * stride, stride * 2, cudaMemcpyDeviceToHost));
        for (uint64_t i = 0; i < stride; ++i) { k_out[i] = __half2float(hk[i]); v_out[i] = __half2float(hv[i]); }
    } else {
        DFL_CUDA(cudaMemcpy(k_out, (const float*)s->k_cache[attn_index] + pos * stride, stride * 4, cudaMemcpyDeviceToHost));
        DFL_CUDA(cudaMemcpy(v_out, (const float*)s->v_cache[attn_index] + pos * stride, stride * 4, cudaMemcpyDeviceToHost));
    }
    return DFL_OK;
}

dfl_status dfl_scratch_create(const dfl_model* m, uint32_t block_size, uint32_t n_capture_layers, dfl_scratch** out) {
    if (!m || !out) return fail(DFL_ERR_BAD_ARG, "scratch_create: null argument");
    *out = nullptr;
    if (block_size < 1 || block_size > MAX_ROWS) return fail(DFL_ERR_BAD_SHAPE, "scratch_create: block_size must be in [1, 16]");
    if (n_capture_layers > DFL_MAX_TARGET_LAYERS) return fail(DFL_ERR_BAD_SHAPE, "scratch_create: too many capture layers");
    DFL_CHECK(use_device(m->device));
    auto* sc = new dfl_scratch();
    sc->m = m;
    sc->block_size = block_size;
    sc->k_layers = n_capture_layers ? n_capture_layers : 1;
    const dfl_arch& a = m->arch;
    const uint64_t H = a.hidden_size, F = a.intermediate_size, V = a.vocab_size;
    const GdnGeom gg = m->gdn_geom();
    const uint64_t q_dim = (uint64_t)a.n_q_heads * a.attn_head_dim, v_dim = (uint64_t)gg.n_v * 128;
    uint64_t part = 0;
    auto upd = [&](const MatGroup& g) { part = std::max<uint64_t>(part, (uint64_t)g.splits * MAX_ROWS * g.total_cols); };
    for (auto& L : m->layers) {
        upd(L.qkv); upd(L.wo); upd(L.in_qkv_z); upd(L.w_out); upd(L.gate_up); upd(L.down); upd(L.moe_gate_up);
        // the experts' and the shared expert's down projections write their partial slices one after the other
        part = std::max<uint64_t>(part, (uint64_t)(L.moe_down.splits + L.moe_down_sh.splits) * MAX_ROWS * H);
    }
    if (m->lm_head.splits > 1) upd(m->lm_head);
    sc->part_floats = part;
    bool ok = true;
    auto alloc = [&](auto** p, size_t bytes) {
        if (!ok) return;
        void* q = nullptr;
        ok = cudaMalloc(&q, bytes ? bytes : 16) == cudaSuccess;
        if (ok) { cudaMemset(q, 0, bytes ? bytes : 16); sc->allocs.push_back(q); }
        *p = reinterpret_cast<std::remove_reference_t<decltype(**p)>*>(q);
    };
    alloc(&sc->x, MAX_ROWS * H * 4);
    alloc(&sc->xn, MAX_ROWS * H * 4);
    alloc(&sc->part, part * 4);
    alloc(&sc->sumsq, (H / GLUE_COLS) * MAX_ROWS * 4);
    const uint64_t chunk = (uint64_t)std::max(act_chunk_bytes(ACT_F16), act_chunk_bytes(ACT_TS));
    alloc(&sc->acts_h, H / TILE_K * chunk);
    const uint64_t f_inner = a.expert_count > 0 ? (uint64_t)m->ep_n * a.expert_feed_forward_length + m->ep_fs : F;
    alloc(&sc->acts_f, f_inner / TILE_K * chunk);
    if (a.expert_count > 0) {
        alloc(&sc->route_logits, (size_t)MAX_ROWS * (a.expert_count + 1) * 4);
        alloc(&sc->route_w, (size_t)MAX_ROWS * a.expert_count * 4);
        alloc(&sc->route_sg, MAX_ROWS * 4);
        alloc(&sc->moe_out, MAX_ROWS * H * 4);
        alloc(&sc->route_idx, (size_t)MAX_ROWS * a.expert_used_count * 4);
        alloc(&sc->moe_tile_map, (size_t)(2 * ((uint64_t)a.expert_count * a.expert_feed_forward_length + a.expert_shared_feed_forward_length) / 128 + 256) * 4);
        alloc(&sc->moe_n_tiles, 16);
        alloc(&sc->moe_kb_map, (size_t)((uint64_t)a.expert_count * a.expert_feed_forward_length / 256 + 64) * 4);
    }
    alloc(&sc->acts_v, std::max(q_dim, v_dim) / TILE_K * chunk);
    alloc(&sc->q_rot, MAX_ROWS * q_dim * 4);
    alloc(&sc->gate, MAX_ROWS * q_dim * 4);
    for (int i = 0; i < m->n_gdn; ++i) {
        float *a0, *a1, *a2, *a3, *a4, *a5;
        alloc(&a0, (size_t)MAX_ROWS * gg.conv_dim() * 4);
        alloc(&a1, (size_t)3 * gg.conv_dim() * 4);
        alloc(&a2, (size_t)MAX_ROWS * gg.n_k * 128 * 4);
        alloc(&a3, (size_t)MAX_ROWS * gg.n_k * 128 * 4);
        alloc(&a4, (size_t)MAX_ROWS * gg.n_v * 128 * 4);
        alloc(&a5, (size_t)MAX_ROWS * 2 * gg.n_v * 4);
        sc->qkv_raw.push_back(a0); sc->conv_pre.push_back(a1); sc->q_n.push_back(a2); sc->k_n.push_back(a3); sc->v.push_back(a4); sc->ab.push_back(a5);
    }
    alloc(&sc->logits, MAX_ROWS * V * 4);
    alloc(&sc->gap, MAX_ROWS * 4);
    alloc(&sc->argmax, MAX_ROWS * 4);
    { uint8_t* am = nullptr; alloc(&am, MAX_ROWS * ARGMAX_PARTS * 16); sc->am_scratch = am; }
    alloc(&sc->capture, (size_t)MAX_ROWS * sc->k_layers * H * 4);
    alloc(&sc->tokens_dev, MAX_ROWS * 4);
    ok = ok && cudaMallocHost(&sc->pinned_i, 2 * MAX_ROWS * 4) == cudaSuccess && cudaMallocHost(&sc->pinned_f, MAX_ROWS * 4) == cudaSuccess;
    if (!ok) {
        std::string why = cudaGetErrorString(cudaGetLastError());
        dfl_scratch_destroy(sc);
        return fail(DFL_ERR_OOM, "scratch_create: allocation failed: " + why);
    }
    cudaDeviceSynchronize();
    *out = sc;
    return DFL_OK;
}

void dfl_scratch_destroy(dfl_scratch* sc) {
    if (!sc) return;
    cudaSetDevice(sc->m->device);
    for (void* p : sc->allocs) cudaFree(p);
    if (sc->pinned_i) cudaFreeHost(sc->pinned_i);
    if (sc->pinned_f) cudaFreeHost(sc->pinned_f);
    if (sc->pinned_logits) cudaFreeHost(sc->pinned_logits);
    if (sc->pinned_order) cudaFreeHost(sc->pinned_order);
    if (sc->order_dev) cudaFree(sc->order_dev);
    if (sc->sort_scratch) cudaFree(sc->sort_scratch);
    delete sc;
}

static dfl_status verify_guards(const dfl_model* m, dfl_session* s, dfl_scratch* sc, const uint32_t* layer_ids, uint32_t n_ids,
                                const int32_t* tokens, uint32_t n, uint32_t start, const char* what) {
    DFL_CHECK(session_guard(m, s, what));
    if (!sc || sc->m != m) return fail(DFL_ERR_BAD_ARG, std::string(what) + ": scratch belongs to another model");
    if (!tokens) return fail(DFL_ERR_BAD_ARG, std::string(what) + ": tokens is null");
    if (n < 1 || n > sc->block_size) return fail(DFL_ERR_BAD_SHAPE, std::string(what) + ": token count must be in [1, block_size]");
    if (n_ids > sc->k_layers || (n_ids && !layer_ids)) return fail(DFL_ERR_BAD_SHAPE, std::string(what) + ": capture layer count exceeds the scratch");
    for (uint32_t k = 0; k < n_ids; ++k)
        if (layer_ids[k] >= m->arch.n_layer) return fail(DFL_ERR_BAD_SHAPE, std::string(what) + ": capture layer id out of range");
    // guard wall of the reference (metal_dflash.rs:9079-9186)
    if (s->kv_n_pos != start) return fail(DFL_ERR_KV_STATE, std::string(what) + ": kv_n_pos " + std::to_string(s->kv_n_pos) + " != start_position " + std::to_string(start));
    if ((uint64_t)start + n > s->kv_capacity) return fail(DFL_ERR_KV_STATE, std::string(what) + ": start_position + n exceeds kv_capacity");
    for (uint32_t i = 0; i < n; ++i)
        if (tokens[i] < 0 || (uint32_t)tokens[i] >= m->arch.vocab_size) return fail(DFL_ERR_BAD_TOKEN, std::string(what) + ": token id out of range");
    return DFL_OK;
}

dfl_status dfl_packed_verify(const dfl_model* m, dfl_session* s, dfl_scratch* sc, const uint32_t* layer_ids, uint32_t n_layer_ids,
                             const int32_t* tokens, uint32_t n, uint32_t start_position, int32_t* argmax_out, float* gap_out,
                             float* logits_host) {
    DFL_CHECK(verify_guards(m, s, sc, layer_ids, n_layer_ids, tokens, n, start_position, "packed_verify"));
    if (!argmax_out) return fail(DFL_ERR_BAD_ARG, "packed_verify: argmax_out is null");
    dfl_status st = verify_core(m, s, sc, layer_ids, n_layer_ids, tokens, n, start_position, true);
    if (st != DFL_OK) { s->poisoned = true; return st; }
    cudaMemcpyAsync(sc->pinned_i + MAX_ROWS, sc->argmax, n * 4, cudaMemcpyDeviceToHost, s->st);
    cudaMemcpyAsync(sc->pinned_f, sc->gap, n * 4, cudaMemcpyDeviceToHost, s->st);
    if (logits_host) cudaMemcpyAsync(logits_host, sc->logits, (size_t)n * m->arch.vocab_size * 4, cudaMemcpyDeviceToHost, s->st);
    if (logits_host && sc->order_host) {
        // the rows' order for the host sampler, produced while the logits travel
        const uint64_t V = m->arch.vocab_size;   // the device buffers exist: dfl_scratch_set_order_host made them
        st = launch_sort_rows_desc(s->st, sc->logits, (int)n, V, V, sc->sort_scratch, sc->order_dev);
        if (st != DFL_OK) { s->poisoned = true; return st; }
        cudaMemcpyAsync(sc->order_host, sc->order_dev, (size_t)n * V * 4, cudaMemcpyDeviceToHost, s->st);
    }
    DFL_CHECK(completion_check(s));
    memcpy(argmax_out, sc->pinned_i + MAX_ROWS, n * 4);
    if (gap_out) memcpy(gap_out, sc->pinned_f, n * 4);
    return DFL_OK;
}

dfl_status dfl_scratch_set_order_host(dfl_scratch* sc, uint32_t* order_host) {
    if (!sc) return fail(DFL_ERR_BAD_ARG, "set_order_host: null scratch");
    sc->order_host = nullptr;
    if (!order_host) return DFL_OK;
    if (!sc->order_dev || !sc->sort_scratch) {   // device side of the ordering, made once per scratch and here, where failing is clean
        DFL_CHECK(use_device(sc->m->device));
        const uint64_t V = sc->m->arch.vocab_size;
        if (!sc->order_dev && cudaMalloc(&sc->order_dev, (size_t)sc->block_size * V * 4) != cudaSuccess) {
            sc->order_dev = nullptr;
            cudaGetLastError();
            return fail(DFL_ERR_OOM, "set_order_host: device order buffer");
        }
        if (!sc->sort_scratch && cudaMalloc(&sc->sort_scratch, sort_rows_scratch_bytes((int)sc->block_size, V)) != cudaSuccess) {
            sc->sort_scratch = nullptr;
            cudaGetLastError();
            return fail(DFL_ERR_OOM, "set_order_host: sort scratch");
        }
    }
    sc->order_host = order_host;
    return DFL_OK;
}

dfl_status dfl_scratch_read_capture(const dfl_scratch* sc, uint32_t n, float* out_host, uint64_t n_floats) {
    if (!sc || !out_host) return fail(DFL_ERR_BAD_ARG, "read_capture: null argument");
    const uint64_t want = (uint64_t)n * sc->k_layers * sc->m->arch.hidden_size;
    if (n > MAX_ROWS || n_floats != want) return fail(DFL_ERR_BAD_SHAPE, "read_capture: size");
    DFL_CHECK(use_device(sc->m->device));
    DFL_CUDA(cudaDeviceSynchronize());
    DFL_CUDA(cudaMemcpy(out_host, sc->capture, want * 4, cudaMemcpyDeviceToHost));
    return DFL_OK;
}


dfl_status dfl_scratch_read_route(const dfl_scratch* sc, uint32_t n, int32_t* idx_out, uint64_t n_idx) {
    if (!sc || !idx_out) return fail(DFL_ERR_BAD_ARG, "read_route: null argument");
    const dfl_arch& a = sc->m->arch;
    if (a.expert_count == 0) return fail(DFL_ERR_UNSUPPORTED, "read_route: the model has no routed experts");
    if (n > MAX_ROWS || n_idx != (uint64_t)n * a.expert_used_count) return fail(DFL_ERR_BAD_SHAPE, "read_route: size");
    DFL_CHECK(use_device(sc->m->device));
    DFL_CUDA(cudaDeviceSynchronize());
    DFL_CUDA(cudaMemcpy(idx_out, sc->route_idx, n_idx * 4, cudaMemcpyDeviceToHost));
    return DFL_OK;
}

// The effective chain length of a call on a scratch made for block_size rows (metal_dflash.rs:9063-9094).
static dfl_status resolve_n_eff(const dfl_scratch* sc, int32_t n_eff_override, const char* what, uint32_t* n_out) {
    if (!sc) return fail(DFL_ERR_BAD_ARG, std::string(what) + ": null scratch");
    const uint32_t n = n_eff_override < 0 ? sc->block_size : (uint32_t)n_eff_override;
    if (n < 1 || n > sc->block_size)
        return fail(DFL_ERR_BAD_SHAPE, std::string(what) + ": n_eff_override resolves to n=" + std::to_string(n) + " which must be in [1, n_block=" +
                                           std::to_string(sc->block_size) + "]");
    *n_out = n;
    return DFL_OK;
}

dfl_status dfl_packed_verify_n_eff(const dfl_model* m, dfl_session* s, dfl_scratch* sc, const uint32_t* layer_ids, uint32_t n_layer_ids,
                                   const int32_t* tokens, uint32_t n_tokens, uint32_t start_position, int32_t n_eff_override,
                                   int32_t* argmax_out, float* gap_out, float* logits_host) {
    uint32_t n = 0;
    DFL_CHECK(resolve_n_eff(sc, n_eff_override, "packed_verify", &n));
    if (n_tokens != n) return fail(DFL_ERR_BAD_SHAPE, "packed_verify: tokens.len()=" + std::to_string(n_tokens) + " != n_eff=" + std::to_string(n));
    return dfl_packed_verify(m, s, sc, layer_ids, n_layer_ids, tokens, n, start_position, argmax_out, gap_out, logits_host);
}

__global__ void wait_probe_kernel(int* err, uint32_t polls) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
        // nobody arrives: the wait runs out after `polls` polls, records why and the kernel returns normally
        mbar_wait_limit(&bar, 0, err, DEV_ERR_WAIT_FLAG, polls);
    }
}

dfl_status dfl_session_probe_wait_timeout(const dfl_model* m, dfl_session* s, uint32_t polls) {
    DFL_CHECK(session_guard(m, s, "probe_wait_timeout"));
    if (polls < 1 || polls > (1u << 16)) return fail(DFL_ERR_BAD_ARG, "probe_wait_timeout: polls must be in [1, 65536]");
    wait_probe_kernel<<<1, 32, 0, s->st>>>(s->err, polls);
    count_launch();
    DFL_CUDA(cudaGetLastError());
    return completion_check(s);
}

}  // extern "C"

namespace dfl {
// The launches of dfl_restore_partial without the wait: the outer loop lets them run under the next draft (the drafter
// never reads the target's recurrent state) and the next verify follows them in stream order.
dfl_status restore_partial_launch(const dfl_model* m, dfl_session* s, dfl_scratch* sc, uint32_t n_keep, uint32_t start_position) {
    DFL_CHECK(session_guard(m, s, "restore_partial"));
    if (!sc || sc->m != m || !sc->have_block) return fail(DFL_ERR_BAD_ARG, "restore_partial: scratch holds no verify block");
    if (start_position != sc->last_start) return fail(DFL_ERR_KV_STATE, "restore_partial: start_position differs from the last verify");
    if (n_keep < 1 || n_keep > sc->last_n) return fail(DFL_ERR_BAD_SHAPE, "restore_partial: n_keep must be in [1, n]");
    if (s->kv_n_pos != sc->last_start + sc->last_n) return fail(DFL_ERR_KV_STATE, "restore_partial: kv_n_pos != start_position + n");
    if (n_keep == sc->last_n) return DFL_OK;  // nothing to undo (metal_dflash.rs:15751)
    const GdnGeom gg = m->gdn_geom();
    int gi = 0;
    for (uint32_t il = 0; il < m->arch.n_layer; ++il) {
        const LayerW& L = m->layers[il];
        if (L.is_attn) continue;
        const int cur = s->ssm_cur[gi];  // advanced state; cur ^ 1 still holds the pre-block state
        dfl_status st = launch_gdn_scan(s->st, gg, s->ssm[cur ^ 1][gi], s->ssm[cur][gi], sc->q_n[gi], sc->k_n[gi], sc->v[gi], sc->ab[gi],
                                        L.dt_bias, L.a_log, (int)n_keep, nullptr, 0, 0, nullptr, nullptr, 0, s->err);
        if (st == DFL_OK) st = launch_gdn_conv_restore(s->st, gg, sc->conv_pre[gi], sc->qkv_raw[gi], (int)n_keep, s->conv[gi]);
        if (st != DFL_OK) { s->poisoned = true; return st; }
        ++gi;
    }
    s->kv_n_pos = start_position + n_keep;  // KV rows beyond stay and are overwritten by the next block
    sc->last_n = n_keep;
    return DFL_OK;
}
}  // namespace dfl

extern "C" {

dfl_status dfl_restore_partial(const dfl_model* m, dfl_session* s, dfl_scratch* sc, uint32_t n_keep, uint32_t start_position) {
    DFL_CHECK(restore_partial_launch(m, s, sc, n_keep, start_position));
    DFL_CUDA(cudaStreamSynchronize(s->st));
    return completion_check(s);
}

dfl_status dfl_restore_partial_n_eff(const dfl_model* m, dfl_session* s, dfl_scratch* sc, uint32_t n_keep, uint32_t start_position,
                                     int32_t n_eff_override) {
    uint32_t n = 0;
    DFL_CHECK(resolve_n_eff(sc, n_eff_override, "restore_partial", &n));
    // the same n_eff as the verify this call undoes (metal_dflash.rs:15662-15666)
    if (sc->have_block && n != sc->last_n_verify) return fail(DFL_ERR_BAD_SHAPE, "restore_partial: n_eff differs from the preceding verify's");
    if (n_keep < 1 || n_keep > n) return fail(DFL_ERR_BAD_SHAPE, "restore_partial: n_keep must be in [1, n_eff=" + std::to_string(n) + "]");
    return dfl_restore_partial(m, s, sc, n_keep, start_position);
}

// ---- session snapshots (SessionSnapshot, metal_forward/session.rs:13-94) ------------------------------------------
struct SnapshotHeader {
    uint32_t magic, header_bytes;
    dfl_snapshot_identity id;
    uint32_t prefix_len, drafter_cols;
    uint32_t drafter_id[3], _pad;   // drafter layer count, K/V row width, sliding window (zeros without a drafter section)
    uint64_t kv_bytes /* each of K and V */, conv_bytes, state_bytes, drafter_bytes;
};
static constexpr uint32_t kSnapshotMagic = 0x534C4644;   // "DFLS"

dfl_status dfl_session_snapshot_identity(const dfl_model* m, const dfl_session* s, dfl_snapshot_identity* out) {
    if (!m || !s || !out || s->m != m) return fail(DFL_ERR_BAD_ARG, "snapshot_identity: bad argument");
    const GdnGeom gg = m->gdn_geom();
    out->layout_version = DFL_SNAPSHOT_LAYOUT_VERSION;
    out->n_attn_layers = (uint32_t)s->k_cache.size();
    out->n_gdn_layers = (uint32_t)s->conv.size();
    out->kv_dim_elements = m->arch.n_kv_heads * m->arch.attn_head_dim;
    out->kv_bytes_per_token = out->kv_dim_elements * (s->kv_f16 ? 2u : 4u);
    out->kv_storage_kind = s->kv_f16 ? 1u : 0u;
    out->gdn_state_elements_per_layer = (uint32_t)((uint64_t)gg.n_v * 128 * 128);
    out->gdn_conv_elements_per_layer = (uint32_t)(3 * gg.conv_dim());
    return DFL_OK;
}

uint64_t dfl_session_snapshot_bytes(const dfl_model* m, const dfl_session* s, const dfl_dsession* ds) {
    dfl_snapshot_identity id;
    if (dfl_session_snapshot_identity(m, s, &id) != DFL_OK) return 0;
    return sizeof(SnapshotHeader) + 2ull * id.n_attn_layers * s->kv_n_pos * id.kv_bytes_per_token +
           (uint64_t)id.n_gdn_layers * (id.gdn_conv_elements_per_layer + id.gdn_state_elements_per_layer) * 4 + (ds ? dsession_snapshot_bytes(ds) : 0);
}

dfl_status dfl_session_snapshot(const dfl_model* m, dfl_session* s, dfl_dsession* ds, void* blob, uint64_t cap, uint64_t* written) {
    DFL_CHECK(session_guard(m, s, "snapshot"));
    if (!blob || !written) return fail(DFL_ERR_BAD_ARG, "snapshot: null argument");
    if (ds && dsession_target(ds) != m) return fail(DFL_ERR_BAD_ARG, "snapshot: drafter session belongs to another model");
    const uint64_t need = dfl_session_snapshot_bytes(m, s, ds);
    if (cap < need) return fail(DFL_ERR_BAD_SHAPE, "snapshot: buffer too small, needs " + std::to_string(need) + " bytes");
    SnapshotHeader h{};
    h.magic = kSnapshotMagic;
    h.header_bytes = sizeof(SnapshotHeader);
    DFL_CHECK(dfl_session_snapshot_identity(m, s, &h.id));
    h.prefix_len = s->kv_n_pos;
    h.kv_bytes = (uint64_t)h.id.n_attn_layers * h.prefix_len * h.id.kv_bytes_per_token;
    h.conv_bytes = (uint64_t)h.id.n_gdn_layers * h.id.gdn_conv_elements_per_layer * 4;
    h.state_bytes = (uint64_t)h.id.n_gdn_layers * h.id.gdn_state_elements_per_layer * 4;
    uint8_t* p = (uint8_t*)blob + sizeof(SnapshotHeader);
    const uint64_t per_layer = (uint64_t)h.prefix_len * h.id.kv_bytes_per_token;
    // packed to the prefix, as position-major rows whatever the session's storage: the unused tail of the cache is not
    // carried, and a snapshot restores into a session of either storage
    void* rows_tmp = nullptr;
    if (s->kv_mode == KV_F16_TILED && per_layer) DFL_CUDA(cudaMalloc(&rows_tmp, per_layer));
    for (int which = 0; which < 2; ++which)
        for (size_t ai = 0; ai < s->k_cache.size(); ++ai, p += per_layer) {
            if (!per_layer) continue;
            const void* src = which ? s->v_cache[ai] : s->k_cache[ai];
            if (rows_tmp) {
                dfl_status cs = launch_kv_tiled_to_rows(s->st, src, which != 0, (int)m->arch.n_kv_heads, 0, h.prefix_len, rows_tmp);
                cudaError_t ce = cs == DFL_OK ? cudaMemcpyAsync(p, rows_tmp, per_layer, cudaMemcpyDeviceToHost, s->st) : cudaSuccess;
                if (ce == cudaSuccess) ce = cudaStreamSynchronize(s->st);   // the staging rows are reused by the next layer
                if (cs != DFL_OK || ce != cudaSuccess) {
                    cudaFree(rows_tmp);
                    DFL_CHECK(cs);
                    DFL_CUDA(ce);
                }
            } else DFL_CUDA(cudaMemcpyAsync(p, src, per_layer, cudaMemcpyDeviceToHost, s->st));
        }
    if (rows_tmp) cudaFree(rows_tmp);
    for (size_t gi = 0; gi < s->conv.size(); ++gi, p += (uint64_t)h.id.gdn_conv_elements_per_layer * 4)
        DFL_CUDA(cudaMemcpyAsync(p, s->conv[gi], (uint64_t)h.id.gdn_conv_elements_per_layer * 4, cudaMemcpyDeviceToHost, s->st));
    for (size_t gi = 0; gi < s->conv.size(); ++gi, p += (uint64_t)h.id.gdn_state_elements_per_layer * 4)
        DFL_CUDA(cudaMemcpyAsync(p, s->ssm[s->ssm_cur[gi]][gi], (uint64_t)h.id.gdn_state_elements_per_layer * 4, cudaMemcpyDeviceToHost, s->st));
    DFL_CUDA(cudaStreamSynchronize(s->st));
    DFL_CHECK(completion_check(s));
    if (ds) {
        h.drafter_bytes = dsession_snapshot_bytes(ds);
        dsession_identity(ds, h.drafter_id);
        DFL_CHECK(dsession_snapshot_write(ds, p, &h.drafter_cols));
        p += h.drafter_bytes;
    }
    memcpy(blob, &h, sizeof(h));
    *written = (uint64_t)(p - (uint8_t*)blob);
    return DFL_OK;
}

dfl_status dfl_session_restore_snapshot(const dfl_model* m, dfl_session* s, dfl_dsession* ds, const void* blob, uint64_t n_bytes) {
    DFL_CHECK(session_guard(m, s, "restore_snapshot"));
    if (!blob) return fail(DFL_ERR_BAD_ARG, "restore_snapshot: null argument");
    if (ds && dsession_target(ds) != m) return fail(DFL_ERR_BAD_ARG, "restore_snapshot: drafter session belongs to another model");
    SnapshotHeader h;
    if (n_bytes < sizeof(h)) return fail(DFL_ERR_BAD_SHAPE, "snapshot header length mismatch");
    memcpy(&h, blob, sizeof(h));
    if (h.magic != kSnapshotMagic || h.header_bytes != sizeof(h)) return fail(DFL_ERR_BAD_ARG, "restore_snapshot: not a session snapshot");
    dfl_snapshot_identity id;
    DFL_CHECK(dfl_session_snapshot_identity(m, s, &id));
    if (memcmp(&id, &h.id, sizeof(id)) != 0) return fail(DFL_ERR_BAD_SHAPE, "snapshot identity mismatch");   // SnapshotValidationError::IdentityMismatch
    if (h.prefix_len > s->kv_capacity)
        return fail(DFL_ERR_KV_STATE, "snapshot prefix length " + std::to_string(h.prefix_len) + " exceeds capacity " + std::to_string(s->kv_capacity));
    const uint64_t per_layer = (uint64_t)h.prefix_len * id.kv_bytes_per_token;
    if (h.kv_bytes != per_layer * id.n_attn_layers || h.conv_bytes != (uint64_t)id.n_gdn_layers * id.gdn_conv_elements_per_layer * 4 ||
        h.state_bytes != (uint64_t)id.n_gdn_layers * id.gdn_state_elements_per_layer * 4 ||
        n_bytes != sizeof(h) + 2 * h.kv_bytes + h.conv_bytes + h.state_bytes + h.drafter_bytes)
        return fail(DFL_ERR_BAD_SHAPE, "snapshot section length mismatch");
    if (ds && h.drafter_bytes == 0 && h.prefix_len > 0) return fail(DFL_ERR_BAD_ARG, "restore_snapshot: the snapshot carries no drafter context");
    if (ds) {   // before the first copy: a refused blob changes nothing
        uint32_t did[3];
        dsession_identity(ds, did);
        if (h.drafter_bytes && memcmp(did, h.drafter_id, sizeof(did)) != 0) return fail(DFL_ERR_BAD_SHAPE, "snapshot drafter identity mismatch");
        DFL_CHECK(dsession_snapshot_validate(ds, h.drafter_cols, h.drafter_bytes));
    }
    const uint8_t* p = (const uint8_t*)blob + sizeof(h);
    void* rows_tmp = nullptr;
    if (s->kv_mode == KV_F16_TILED && per_layer) DFL_CUDA(cudaMalloc(&rows_tmp, per_layer));
    for (int which = 0; which < 2; ++which)
        for (size_t ai = 0; ai < s->k_cache.size(); ++ai, p += per_layer) {
            if (!per_layer) continue;
            void* dst = which ? s->v_cache[ai] : s->k_cache[ai];
            if (rows_tmp) {
                cudaError_t ce = cudaMemcpyAsync(rows_tmp, p, per_layer, cudaMemcpyHostToDevice, s->st);
                dfl_status cs = ce == cudaSuccess ? launch_kv_rows_to_tiled(s->st, rows_tmp, which != 0, (int)m->arch.n_kv_heads, 0, h.prefix_len, dst) : DFL_OK;
                if (ce == cudaSuccess) ce = cudaStreamSynchronize(s->st);
                if (cs != DFL_OK || ce != cudaSuccess) {
                    cudaFree(rows_tmp);
                    s->poisoned = true;   // part of the state has been overwritten
                    DFL_CHECK(cs);
                    DFL_CUDA(ce);
                }
            } else DFL_CUDA(cudaMemcpyAsync(dst, p, per_layer, cudaMemcpyHostToDevice, s->st));
        }
    if (rows_tmp) cudaFree(rows_tmp);
    for (size_t gi = 0; gi < s->conv.size(); ++gi, p += (uint64_t)id.gdn_conv_elements_per_layer * 4)
        DFL_CUDA(cudaMemcpyAsync(s->conv[gi], p, (uint64_t)id.gdn_conv_elements_per_layer * 4, cudaMemcpyHostToDevice, s->st));
    for (size_t gi = 0; gi < s->conv.size(); ++gi, p += (uint64_t)id.gdn_state_elements_per_layer * 4)
        DFL_CUDA(cudaMemcpyAsync(s->ssm[s->ssm_cur[gi]][gi], p, (uint64_t)id.gdn_state_elements_per_layer * 4, cudaMemcpyHostToDevice, s->st));
    DFL_CUDA(cudaStreamSynchronize(s->st));
    s->kv_n_pos = h.prefix_len;
    if (ds) DFL_CHECK(dsession_snapshot_read(ds, p, h.drafter_cols, h.drafter_bytes));
    return completion_check(s);
}

dfl_status dfl_restore_pre_block(const dfl_model* m, dfl_session* s, dfl_scratch* sc, uint32_t start_position) {
    DFL_CHECK(session_guard(m, s, "restore_pre_block"));
    if (!sc || sc->m != m || !sc->have_block) return fail(DFL_ERR_BAD_ARG, "restore_pre_block: scratch holds no verify block");
    if (start_position != sc->last_start) return fail(DFL_ERR_KV_STATE, "restore_pre_block: start_position differs from the last verify");
    const GdnGeom gg = m->gdn_geom();
    for (size_t gi = 0; gi < s->conv.size(); ++gi) {
        s->ssm_cur[gi] ^= 1;
        DFL_CUDA(cudaMemcpyAsync(s->conv[gi], sc->conv_pre[gi], (size_t)3 * gg.conv_dim() * 4, cudaMemcpyDeviceToDevice, s->st));
    }
    s->kv_n_pos = start_position;
    sc->have_block = false;
    DFL_CUDA(cudaStreamSynchronize(s->st));
    return completion_check(s);
}

dfl_status dfl_single_token(const dfl_model* m, dfl_session* s, dfl_scratch* sc, const uint32_t* layer_ids, uint32_t n_layer_ids,
                            int32_t token, uint32_t position, float* logits_host, float* hidden_host) {
    DFL_CHECK(verify_guards(m, s, sc, layer_ids, n_layer_ids, &token, 1, position, "single_token"));
    dfl_status st = verify_core(m, s, sc, layer_ids, n_layer_ids, &token, 1, position, true);
    if (st != DFL_OK) { s->poisoned = true; return st; }
    if (logits_host) cudaMemcpyAsync(logits_host, sc->logits, (size_t)m->arch.vocab_size * 4, cudaMemcpyDeviceToHost, s->st);
    if (hidden_host && n_layer_ids)   // [n_layer_ids][H]: the caller's slots, whatever the scratch was sized for
        cudaMemcpyAsync(hidden_host, sc->capture, (size_t)n_layer_ids * m->arch.hidden_size * 4, cudaMemcpyDeviceToHost, s->st);
    return completion_check(s);
}

}  // extern "C"
