// Prompt prefill through the packed path and the DFlash outer loop
// (reference: prefill_tokens_with_multi_hidden, crates/qwen-llm/src/metal_dflash.rs:10779-10787;
// generate_dflash, crates/qwen-cli/src/qwen/dflash.rs:484-1263).
#include <chrono>
#include <cstring>
#include <vector>

#include "model.cuh"

struct dfl_dsession;
struct dfl_drafter;
namespace dfl {
dfl_status draft_core(dfl_dsession* ds, int32_t carry, uint32_t noise_start, bool topk);
dfl_status draft_block_topk(dfl_dsession* ds, int32_t carry, uint32_t noise_start_pos, int32_t* out_tokens);
dfl_status restore_partial_launch(const dfl_model* m, dfl_session* s, dfl_scratch* sc, uint32_t n_keep, uint32_t start_position);
void dsession_set_after_enqueue(dfl_dsession* ds, void (*fn)(void*), void* arg);
}
// accessors implemented next to the drafter session (drafter.cu)
extern "C" {
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
void dfl_dsession_view_get(dfl_dsession* ds, dfl_dsession_view* out);
}

using namespace dfl;

static double now_ms() {
    return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

extern "C" {

dfl_status dfl_prefill(const dfl_model* m, dfl_session* s, dfl_scratch* sc, const uint32_t* layer_ids, uint32_t n_layer_ids, const int32_t* ids,
                       uint64_t n, uint32_t start_position, dfl_dsession* feed_drafter, float* hidden_host, float* last_logits_host) {
    DFL_CHECK(session_guard(m, s, "prefill"));
    if (!sc || sc->m != m || !ids || n == 0) return fail(DFL_ERR_BAD_ARG, "prefill: bad argument");
    if (s->kv_n_pos != start_position) return fail(DFL_ERR_KV_STATE, "prefill: kv_n_pos != start_position");
    if ((uint64_t)start_position + n > s->kv_capacity) return fail(DFL_ERR_KV_STATE, "prefill: prompt does not fit the KV capacity");
    if (n_layer_ids > sc->k_layers || (n_layer_ids && !layer_ids)) return fail(DFL_ERR_BAD_SHAPE, "prefill: capture layer count exceeds the scratch");
    for (uint32_t k = 0; k < n_layer_ids; ++k)
        if (layer_ids[k] >= m->arch.n_layer) return fail(DFL_ERR_BAD_SHAPE, "prefill: capture layer id out of range");
    // the drafter consumes every slot of a captured row: a shorter id list would feed it slots no layer wrote
    if (feed_drafter && n_layer_ids != sc->k_layers) return fail(DFL_ERR_BAD_SHAPE, "prefill: feeding the drafter needs one capture layer per scratch slot");
    for (uint64_t i = 0; i < n; ++i)
        if (ids[i] < 0 || (uint32_t)ids[i] >= m->arch.vocab_size) return fail(DFL_ERR_BAD_TOKEN, "prefill: token id out of range");
    const uint64_t KH = (uint64_t)sc->k_layers * m->arch.hidden_size;
    const uint32_t bs = sc->block_size;
    for (uint64_t off = 0; off < n; off += bs) {
        const uint32_t nb = (uint32_t)std::min<uint64_t>(bs, n - off);
        const bool last = off + nb == n;
        dfl_status st = verify_core(m, s, sc, layer_ids, n_layer_ids, ids + off, nb, start_position + (uint32_t)off, last && last_logits_host != nullptr);
        if (st != DFL_OK) { s->poisoned = true; return st; }
        if (hidden_host && n_layer_ids)
            cudaMemcpyAsync(hidden_host + off * KH, sc->capture, (size_t)nb * KH * 4, cudaMemcpyDeviceToHost, s->st);
        if (last && last_logits_host)
            cudaMemcpyAsync(last_logits_host, sc->logits + (uint64_t)(nb - 1) * m->arch.vocab_size, (size_t)m->arch.vocab_size * 4,
                            cudaMemcpyDeviceToHost, s->st);
        DFL_CHECK(session_drain(s));
        if (feed_drafter) DFL_CHECK(dfl_dsession_append_from_scratch(feed_drafter, sc, 0, nb, start_position + (uint32_t)off));
    }
    dfl_status st = check_dev_err(s->st, s->err);
    if (st != DFL_OK) s->poisoned = true;
    return st;
}

dfl_status dfl_generate(const dfl_model* m, dfl_session* s, dfl_scratch* sc, dfl_dsession* ds, dfl_sampler* sampler, const float* first_logits,
                        const dfl_generate_params* params, int32_t* tokens_out, uint32_t* n_out, dfl_generate_stats* stats) {
    DFL_CHECK(session_guard(m, s, "generate"));
    if (!sc || !ds || !sampler || !first_logits || !params || !tokens_out || !n_out) return fail(DFL_ERR_BAD_ARG, "generate: null argument");
    if (params->max_tokens == 0) return fail(DFL_ERR_BAD_ARG, "generate: max_tokens must be >= 1");
    dfl_dsession_view dv;
    dfl_dsession_view_get(ds, &dv);
    if (dv.target != m || sc->m != m) return fail(DFL_ERR_BAD_ARG, "generate: handles belong to different models");
    if (sc->k_layers != dv.n_target_layers) return fail(DFL_ERR_BAD_SHAPE, "generate: scratch capture layer count differs from the drafter's");
    const uint32_t N = dv.block_size, V = m->arch.vocab_size;
    if (sc->block_size < N) return fail(DFL_ERR_BAD_SHAPE, "generate: scratch block size is smaller than the drafter block");
    dfl_generate_stats st{};
    const double wall0 = now_ms();
    int32_t carry = 0;
    uint64_t idx = 0;
    DFL_CHECK(dfl_sampler_sample(sampler, first_logits, V, &carry, &idx));
    dfl_sampling_config scfg;
    dfl_sampler_get_config(sampler, &scfg);
    const bool sampled = scfg.temperature > 0.0f;
    dfl_sampler* proposal_sampler = nullptr;
    if (sampled && params->sparse_proposals) {
        dfl_sampling_config pc{scfg.temperature, 0, 1.0f, 0.0f, scfg.seed ^ 0x44464c4153483251ull};  // qwen/dflash.rs:91
        DFL_CHECK(dfl_sampler_create(&pc, &proposal_sampler));
    }
    // the block's logits for the host sampler: pinned (the 16 x vocab copy runs at link speed) and kept with the scratch,
    // since pinning and unpinning 10 MB costs far more than a step
    if (sampled && !sc->pinned_logits && cudaMallocHost(&sc->pinned_logits, (size_t)sc->block_size * V * 4) != cudaSuccess) {
        sc->pinned_logits = nullptr;
        if (proposal_sampler) dfl_sampler_destroy(proposal_sampler);
        return fail(DFL_ERR_OOM, "generate: pinned logits buffer");
    }
    struct { float* p; float* data() const { return p; } } logits_host{sc->pinned_logits};
    // rows ordered on the device: the order lands beside the logits and the sampler is told where (cleared on every exit)
    const bool device_order = sampled && params->device_row_order;
    if (device_order) {
        if (!sc->pinned_order && cudaMallocHost(&sc->pinned_order, (size_t)sc->block_size * V * 4) != cudaSuccess) {
            sc->pinned_order = nullptr;
            if (proposal_sampler) dfl_sampler_destroy(proposal_sampler);
            return fail(DFL_ERR_OOM, "generate: pinned row-order buffer");
        }
        const dfl_status os = dfl_scratch_set_order_host(sc, sc->pinned_order);
        if (os != DFL_OK) {
            if (proposal_sampler) dfl_sampler_destroy(proposal_sampler);
            return os;
        }
        dfl_sampler_set_row_order(sampler, sc->pinned_logits, sc->pinned_order, sc->block_size, V);
    }
    auto is_stop = [&](int32_t t) {
        for (uint32_t i = 0; i < params->n_stop_ids; ++i)
            if (params->stop_ids[i] == t) return true;
        return false;
    };
    std::vector<int32_t> tokens;
    tokens.reserve(params->max_tokens);
    dfl_status rc = DFL_OK;
    int32_t draft[MAX_ROWS], verify_in[MAX_ROWS], argmax[MAX_ROWS];
    float gap[MAX_ROWS];
    // A partial-accept rollback is launched without a wait and runs under the next draft; what is counted as restore
    // time is the part of it that outlasts that draft (all of it when no draft runs).
    bool restore_pending = false;
    // The rollback itself is queued late: behind the next draft's launches when a draft follows (the host then spends
    // its launch time on the drafter first and the GPU is not left waiting), else right before whatever comes next.
    struct Deferred {
        bool on = false;
        uint32_t n_keep = 0, position = 0;
        dfl_status rc = DFL_OK;
        const dfl_model* m;
        dfl_session* s;
        dfl_scratch* sc;
        bool* pending;
        uint32_t* calls;
        void launch() {
            if (!on) return;
            on = false;
            cudaEventRecord(s->ev0, s->st);
            rc = n_keep == 0 ? dfl_restore_pre_block(m, s, sc, position) : restore_partial_launch(m, s, sc, n_keep, position);
            cudaEventRecord(s->ev1, s->st);
            if (rc == DFL_OK) { *pending = true; ++*calls; }
        }
        static void hook(void* self) { static_cast<Deferred*>(self)->launch(); }
    } deferred;
    deferred.m = m; deferred.s = s; deferred.sc = sc; deferred.pending = &restore_pending; deferred.calls = &st.restore_calls;
    auto settle_restore = [&](bool draft_ran) {
        deferred.launch();
        if (deferred.rc != DFL_OK && rc == DFL_OK) rc = deferred.rc;
        if (!restore_pending) return;
        restore_pending = false;
        cudaEventSynchronize(s->ev1);
        float ms = 0;
        if (draft_ran) cudaEventElapsedTime(&ms, dv.ev1, s->ev1);
        else cudaEventElapsedTime(&ms, s->ev0, s->ev1);
        if (ms > 0) st.restore_ms += ms;
    };
    for (;;) {
        tokens.push_back(carry);
        if (is_stop(carry)) break;
        if (tokens.size() == params->max_tokens) break;
        // a rollback that is still to be queued has not moved the session's position yet
        const uint32_t position = deferred.on ? deferred.position + deferred.n_keep : s->kv_n_pos;
        const uint32_t remaining_ctx = s->kv_capacity - position;
        if (remaining_ctx < N) {
            // off step (qwen/dflash.rs:629-637): exact single-token decode keeps the loop going near the capacity edge
            if (remaining_ctx == 0) break;
            settle_restore(false);
            std::vector<float> l(V);
            rc = dfl_single_token(m, s, sc, dv.target_layer_ids, dv.n_target_layers, carry, position, l.data(), nullptr);
            if (rc != DFL_OK) break;
            rc = dfl_sampler_sample(sampler, l.data(), V, &carry, &idx);
            if (rc != DFL_OK) break;
            continue;
        }
        // ---- draft ----
        const int32_t* replay = nullptr;
        if (params->replay_history && !proposal_sampler) {  // dflash_prefix_replay_drafts, qwen/dflash.rs:351-360 (one-hot coupling when sampled)
            const size_t emitted = tokens.size();
            if (emitted + (N - 1) <= params->n_replay_history &&
                (params->replay_unchecked || std::memcmp(params->replay_history, tokens.data(), emitted * 4) == 0))
                replay = params->replay_history + emitted;
        }
        std::vector<int32_t> prop_tok;
        std::vector<uint32_t> prop_off;
        std::vector<int32_t> prop_ct;
        std::vector<double> prop_cw;
        if (replay) {
            if (params->replay_runs_drafter) {
                int32_t discard[MAX_ROWS];
                cudaEventRecord(dv.ev0, dv.st);
                if (deferred.on) dsession_set_after_enqueue(ds, &Deferred::hook, &deferred);
                rc = dfl_draft_block(ds, carry, position, discard, nullptr);
                dsession_set_after_enqueue(ds, nullptr, nullptr);
                cudaEventRecord(dv.ev1, dv.st);
                if (rc != DFL_OK) break;
                cudaEventSynchronize(dv.ev1);
                float ms = 0;
                cudaEventElapsedTime(&ms, dv.ev0, dv.ev1);
                st.draft_ms += ms;
                ++st.drafter_calls;
            }
            draft[0] = carry;
            for (uint32_t i = 1; i < N; ++i) draft[i] = replay[i - 1];
        } else {
            cudaEventRecord(dv.ev0, dv.st);
            const bool selector_sampled = proposal_sampler && dv.has_selector;
            uint32_t sel_off[DFL_MAX_BLOCK];
            int32_t sel_ct[DFL_MAX_BLOCK * 16];
            double sel_cw[DFL_MAX_BLOCK * 16];
            if (deferred.on) dsession_set_after_enqueue(ds, &Deferred::hook, &deferred);
            if (selector_sampled) rc = dfl_draft_block_sampled(ds, carry, position, proposal_sampler, draft, sel_off, sel_ct, sel_cw);
            else if (proposal_sampler) rc = draft_block_topk(ds, carry, position, draft);
            else rc = dfl_draft_block(ds, carry, position, draft, nullptr);
            dsession_set_after_enqueue(ds, nullptr, nullptr);
            cudaEventRecord(dv.ev1, dv.st);
            if (rc != DFL_OK) break;
            cudaEventSynchronize(dv.ev1);
            float ms = 0;
            cudaEventElapsedTime(&ms, dv.ev0, dv.ev1);
            st.draft_ms += ms;
            ++st.drafter_calls;
            if (selector_sampled) {   // draft_block_sampled, metal_dflash.rs:17268-17415
                prop_off.push_back(0);
                for (uint32_t pos = 1; pos < N; ++pos) {
                    prop_tok.push_back(draft[pos]);
                    for (uint32_t k = sel_off[pos - 1]; k < sel_off[pos]; ++k) { prop_ct.push_back(sel_ct[k]); prop_cw.push_back(sel_cw[k]); }
                    prop_off.push_back((uint32_t)prop_ct.size());
                }
            } else if (proposal_sampler) {
                // a drafter without a selector: the same sparse proposals from the device's top-16 with the pair term absent
                int32_t top_ids[DFL_MAX_BLOCK * 16];
                float top_vals[DFL_MAX_BLOCK * 16];
                rc = dfl_dsession_read_selector(ds, top_ids, top_vals, nullptr);
                if (rc != DFL_OK) break;
                prop_off.push_back(0);
                for (uint32_t pos = 1; pos < N && rc == DFL_OK; ++pos) {
                    const int32_t* ids = top_ids + pos * 16;
                    float vals[16];
                    int cnt = 0;
                    while (cnt < 16 && ids[cnt] >= 0) { vals[cnt] = top_vals[pos * 16 + cnt]; ++cnt; }
                    int32_t sel = 0;
                    int32_t dt[16];
                    double dw[16];
                    uint64_t count = 0, ci = 0;
                    double total = 0;
                    rc = dfl_sampler_sample_with_distribution(proposal_sampler, vals, (uint64_t)cnt, &sel, &ci, dt, dw, 16, &count, &total);
                    if (rc != DFL_OK) break;
                    draft[pos] = ids[sel];
                    prop_tok.push_back(ids[sel]);
                    for (uint64_t k = 0; k < count; ++k)
                        if (dw[k] > 0.0) { prop_ct.push_back(ids[dt[k]]); prop_cw.push_back(dw[k]); }
                    prop_off.push_back((uint32_t)prop_ct.size());
                }
                if (rc != DFL_OK) break;
            }
        }
        ++st.spec_steps;
        settle_restore(!replay || params->replay_runs_drafter);
        if (rc != DFL_OK) break;
        // ---- packed verify of [carry, drafts...] ----
        verify_in[0] = carry;
        for (uint32_t i = 1; i < N; ++i) verify_in[i] = draft[i];
        cudaEventRecord(s->ev0, s->st);
        rc = dfl_packed_verify(m, s, sc, dv.target_layer_ids, dv.n_target_layers, verify_in, N, position, argmax, gap, sampled ? logits_host.data() : nullptr);
        cudaEventRecord(s->ev1, s->st);
        if (rc != DFL_OK) break;
        cudaEventSynchronize(s->ev1);
        {
            float ms = 0;
            cudaEventElapsedTime(&ms, s->ev0, s->ev1);
            st.verify_ms += ms;
        }
        ++st.verify_calls;
        st.drafts_scored += N - 1;
        // ---- accept prefix ----
        const double t_acc = now_ms();
        dfl_accept_decision dec;
        const uint64_t budget = params->max_tokens - tokens.size();
        if (sampled) {
            dfl_sparse_proposals sp{N - 1, prop_tok.data(), prop_off.data(), prop_ct.data(), prop_cw.data()};
            rc = dfl_accept_prefix(verify_in, N, logits_host.data(), (uint64_t)N * V, V, proposal_sampler ? &sp : nullptr, sampler, budget, params->stop_ids,
                                   params->n_stop_ids, &dec);
            if (rc != DFL_OK) break;
        } else {
            // greedy prefix (qwen/dflash.rs:838-852): accept while draft == target argmax
            std::memset(&dec, 0, sizeof(dec));
            uint32_t a = 0;
            int stop = DFL_STOP_NONE;
            while (a < N - 1 && verify_in[a + 1] == argmax[a]) {
                dec.accepted_drafts[a] = verify_in[a + 1];
                ++a;
                if (is_stop(verify_in[a])) { stop = DFL_STOP_EOS; break; }
                if (a == budget) { stop = DFL_STOP_TOKEN_LIMIT; break; }
            }
            dec.n_accepted = a;
            dec.stop_reason = stop;
            dec.retain_input_count = stop ? a : a + 1;
            if (!stop) {
                if (argmax[a] < 0) { rc = fail(DFL_ERR_SAMPLING, "DFlash target row " + std::to_string(a) + ": logit is NaN"); break; }
                dec.next_carry = argmax[a];
                dec.next_carry_kind = a == N - 1 ? DFL_CARRY_BONUS : DFL_CARRY_CORRECTION;
            }
        }
        st.accept_ms += now_ms() - t_acc;
        const uint32_t n_keep = dec.retain_input_count;
        // ---- margin guard (qwen/dflash.rs:859-1057): count committed rows whose gap is below the margin ----
        if (!sampled && params->verify_margin > 0.f) {
            uint32_t flagged = 0;
            for (uint32_t r = 0; r < n_keep; ++r) flagged += gap[r] < params->verify_margin;
            st.committed_rows += n_keep;
            st.margin_rows += flagged;
            if (flagged) ++st.fallback_steps;
        }
        // ---- append captured hiddens of the committed rows, then roll the target back ----
        const double t_app = now_ms();
        if (n_keep > 0) {
            rc = dfl_dsession_append_from_scratch(ds, sc, 0, n_keep, position);
            if (rc != DFL_OK) break;
        }
        st.append_ms += now_ms() - t_app;
        if (n_keep < N) {
            deferred.on = true;
            deferred.n_keep = n_keep;
            deferred.position = position;
        }
        st.accepted_drafts += dec.n_accepted;
        bool done = false;
        for (uint32_t i = 0; i < dec.n_accepted; ++i) {
            tokens.push_back(dec.accepted_drafts[i]);
            if (tokens.size() == params->max_tokens) done = true;
        }
        if (dec.stop_reason != DFL_STOP_NONE || done) break;
        carry = dec.next_carry;
    }
    if (proposal_sampler) dfl_sampler_destroy(proposal_sampler);
    if (device_order) {
        dfl_scratch_set_order_host(sc, nullptr);
        dfl_sampler_set_row_order(sampler, nullptr, nullptr, 0, 0);
    }
    settle_restore(false);
    if (rc == DFL_OK) {   // nothing of this call is left in flight when it returns
        if (cudaStreamSynchronize(s->st) != cudaSuccess) rc = fail(DFL_ERR_CUDA, "generate: stream synchronize failed");
        else rc = check_dev_err(s->st, s->err);
        if (rc != DFL_OK) s->poisoned = true;
    }
    const uint32_t n_emit = (uint32_t)std::min<size_t>(tokens.size(), params->max_tokens);
    std::memcpy(tokens_out, tokens.data(), (size_t)n_emit * 4);
    *n_out = n_emit;
    st.tokens_emitted = n_emit;
    st.wall_ms = now_ms() - wall0;
    if (stats) *stats = st;
    return rc;
}

}  // extern "C"
