// TEST INFRASTRUCTURE — CPU oracle, never linked into or called by the product.
//
// Scalar f32 restatement of the reference's CPU forward pass
// (crates/qwen-llm/src/forward.rs): `single_token_capture_layers` (:173-220),
// `dflash_draft` (:380-662), `ffn` (:725-747), `ffn_moe` (:749-824), `attn_step`
// (:834-932), `gdn_step` (:940-1107), `KvCache` (:1133-1240) and the math
// primitives (:1244-1371).  Loop order and operation order follow the reference so
// that every sum is accumulated in the same sequence.  Weights are dequantised once
// and cached (the reference re-dequantises per call, forward.rs:679-682; the values
// are identical).  OpenMP parallelises over output rows only, which leaves each
// row's summation order unchanged.
//
// Parity status: the primitives are pinned by forward.rs:1377-1414; the reference
// has no golden vectors for whole-model logits that can run without its model files
// (forward.rs:1416-1886 need GGUFs), so end-to-end logits parity is "parity unpinned"
// for the full forward: it rests on this restatement and on its agreement, token by
// token, with a second restatement written separately in numpy over other block
// decoders (oracle/forward_np.py, tests/test_oracle_twin.py).
#pragma once
#include <algorithm>
#include <cmath>
#include <map>
#include <memory>
#include <string>
#include <utility>
#include <vector>

#include "../include/dflash_b200.h"
#include "quants.hpp"

namespace oracle {

constexpr float RMS_EPS = 1e-6f;  // forward.rs:1244

// ---- primitives (forward.rs:1256-1371) -----------------------------------
inline std::vector<float> rms_norm(const float* x, size_t n, const float* w, float eps) {
    float ss = 0.f;
    for (size_t i = 0; i < n; ++i) ss += x[i] * x[i];
    const float mean_sq = ss / (float)n;
    const float scale = 1.0f / std::sqrt(mean_sq + eps);
    std::vector<float> y(n);
    for (size_t i = 0; i < n; ++i) y[i] = x[i] * scale * w[i];
    return y;
}
inline void l2_norm_in_place(float* x, size_t n, float eps) {
    float sq = 0.f;
    for (size_t i = 0; i < n; ++i) sq += x[i] * x[i];
    const float scale = 1.0f / std::max(std::sqrt(sq), eps);
    for (size_t i = 0; i < n; ++i) x[i] *= scale;
}
inline float silu(float x) { return x / (1.0f + std::exp(-x)); }
inline float sigmoid(float x) { return 1.0f / (1.0f + std::exp(-x)); }
inline float softplus(float x) {
    if (x > 20.0f) return x;
    if (x < -20.0f) return std::exp(x);
    return std::log(1.0f + std::exp(x));
}
inline void softmax_in_place(float* x, size_t n) {
    float mx = -INFINITY;
    for (size_t i = 0; i < n; ++i) mx = std::max(mx, x[i]);
    float sum = 0.f;
    for (size_t i = 0; i < n; ++i) { x[i] = std::exp(x[i] - mx); sum += x[i]; }
    const float inv = 1.0f / sum;
    for (size_t i = 0; i < n; ++i) x[i] *= inv;
}
// y[o] = sum_i x[i] * w[o*n_in + i], sequential in i (forward.rs:1321-1334).
inline std::vector<float> mat_vec(const float* w, size_t n_in, size_t n_out, const float* x) {
    std::vector<float> y(n_out);
#pragma omp parallel for schedule(static) if (n_in * n_out > (1u << 18))
    for (long o = 0; o < (long)n_out; ++o) {
        const float* row = w + (size_t)o * n_in;
        float s = 0.f;
        for (size_t i = 0; i < n_in; ++i) s += x[i] * row[i];
        y[o] = s;
    }
    return y;
}
// NeoX partial RoPE (forward.rs:1347-1371).
inline void rope_in_place(float* buf, size_t n_heads, size_t head_dim, size_t n_rot, uint32_t position,
                          float theta_base) {
    const float pos = (float)position;
    const size_t half = n_rot / 2;
    for (size_t hi = 0; hi < n_heads; ++hi) {
        const size_t off = hi * head_dim;
        for (size_t i = 0; i < half; ++i) {
            const float exponent = (float)(2 * i) / (float)n_rot;
            const float freq = pos / std::pow(theta_base, exponent);
            const float s = std::sin(freq), c = std::cos(freq);
            const float a = buf[off + i], b = buf[off + i + half];
            buf[off + i] = a * c - b * s;
            buf[off + i + half] = a * s + b * c;
        }
    }
}

// ---- tensors ------------------------------------------------------------
struct Tensor {
    int32_t dtype = 0;
    std::vector<uint64_t> shape;
    std::vector<uint8_t> bytes;
    mutable std::vector<float> f32;  // dequantised cache
    uint64_t n_elements() const { uint64_t n = 1; for (auto d : shape) n *= d; return n; }
    const float* deq() const {
        if (f32.empty()) {
            f32.resize(n_elements());
            dequant_to_f32(dtype, bytes.data(), n_elements(), f32.data());
        }
        return f32.data();
    }
    void drop_cache() const { std::vector<float>().swap(f32); }
};

struct TensorTable {
    std::map<std::string, Tensor> t;
    void add(const dfl_tensor& d) {
        Tensor x;
        x.dtype = d.dtype;
        x.shape.assign(d.shape, d.shape + d.n_dims);
        x.bytes.assign((const uint8_t*)d.data, (const uint8_t*)d.data + d.n_bytes);
        t[d.name] = std::move(x);
    }
    const Tensor& need(const std::string& name) const {
        auto it = t.find(name);
        if (it == t.end()) throw std::runtime_error("oracle: missing tensor " + name);
        return it->second;
    }
    const Tensor* find(const std::string& name) const {
        auto it = t.find(name);
        return it == t.end() ? nullptr : &it->second;
    }
};

// ---- state --------------------------------------------------------------
struct State {
    std::vector<std::vector<float>> conv;  // [n_gdn][(kernel-1) * conv_dim], time-major rows
    std::vector<std::vector<float>> ssm;   // [n_gdn][n_v * hd * hd]  (head, dv, dk)
    // KvCache (forward.rs:1133-1240): per layer [pos][kv_head][head_dim]
    std::vector<std::vector<float>> k, v;
    std::vector<size_t> n_pos;
    size_t capacity = 0;
    bool kv_f16 = false;  // round K/V to binary16 at append (the GPU cache layout)
};

struct Model {
    dfl_arch arch{};
    TensorTable tt;
    bool is_attn(uint32_t il) const {  // model.rs:78-86
        const uint32_t iv = std::max(arch.full_attention_interval, 1u);
        return il % iv == iv - 1;
    }
    size_t n_gdn() const { size_t n = 0; for (uint32_t i = 0; i < arch.n_layer; ++i) n += !is_attn(i); return n; }
    const Tensor& lm_head() const {
        if (auto* t = tt.find("output.weight")) return *t;
        return tt.need("token_embd.weight");  // tied embeddings, loader.rs:445
    }
    State fresh_state(size_t kv_capacity, bool kv_f16) const {
        State s;
        const size_t conv_dim = (2 * arch.gdn_n_k_heads + arch.gdn_n_v_heads) * (size_t)arch.gdn_head_dim;
        const size_t ng = n_gdn();
        s.conv.assign(ng, std::vector<float>(conv_dim * (arch.gdn_conv_kernel - 1), 0.f));
        s.ssm.assign(ng, std::vector<float>((size_t)arch.gdn_head_dim * arch.gdn_head_dim * arch.gdn_n_v_heads, 0.f));
        s.k.assign(arch.n_layer, {});
        s.v.assign(arch.n_layer, {});
        s.n_pos.assign(arch.n_layer, 0);
        s.capacity = kv_capacity;
        s.kv_f16 = kv_f16;
        return s;
    }

    std::string blk(uint32_t il, const char* suffix) const { return "blk." + std::to_string(il) + "." + suffix; }

    std::vector<float> embed_token(int32_t id) const {  // forward.rs:666-677
        const Tensor& e = tt.need("token_embd.weight");
        const size_t h = arch.hidden_size;
        // only the needed row is decoded; rows are block aligned
        uint64_t blk_n, blk_b;
        storage_layout(e.dtype, blk_n, blk_b);
        const size_t row_bytes = h / blk_n * blk_b;
        std::vector<float> out(h);
        dequant_to_f32(e.dtype, e.bytes.data() + (size_t)id * row_bytes, h, out.data());
        return out;
    }

    // forward.rs:725-747
    std::vector<float> ffn(uint32_t il, const float* x) const {
        if (arch.expert_count > 0) return ffn_moe(il, x);
        const size_t h = arch.hidden_size, f = arch.intermediate_size;
        auto gated = mat_vec(tt.need(blk(il, "ffn_gate.weight")).deq(), h, f, x);
        auto upped = mat_vec(tt.need(blk(il, "ffn_up.weight")).deq(), h, f, x);
        std::vector<float> hidden(f);
        for (size_t i = 0; i < f; ++i) hidden[i] = silu(gated[i]) * upped[i];
        return mat_vec(tt.need(blk(il, "ffn_down.weight")).deq(), f, h, hidden.data());
    }

    // forward.rs:749-824
    mutable std::vector<int32_t> last_route;  // expert ids chosen by the most recent ffn_moe call
    std::vector<float> ffn_moe(uint32_t il, const float* x) const {
        const size_t h = arch.hidden_size, n_expert = arch.expert_count;
        const size_t n_used = std::min(arch.expert_used_count, arch.expert_count);
        const size_t f_exp = arch.expert_feed_forward_length, f_sh = arch.expert_shared_feed_forward_length;
        auto probs = mat_vec(tt.need(blk(il, "ffn_gate_inp.weight")).deq(), h, n_expert, x);
        softmax_in_place(probs.data(), n_expert);
        std::vector<std::pair<size_t, float>> ranked(n_expert);
        for (size_t i = 0; i < n_expert; ++i) ranked[i] = {i, probs[i]};
        std::stable_sort(ranked.begin(), ranked.end(), [](const auto& a, const auto& b) {
            if (a.second > b.second) return true;   // probability descending
            if (a.second < b.second) return false;
            return a.first < b.first;               // then index ascending
        });
        ranked.resize(n_used);
        float weight_sum = 0.f;
        for (auto& r : ranked) weight_sum += r.second;
        weight_sum = std::max(weight_sum, 6.103515625e-05f);  // 2^-14, bits 0x38800000
        std::vector<float> out(h, 0.f);
        const Tensor& ge = tt.need(blk(il, "ffn_gate_exps.weight"));
        const Tensor& ue = tt.need(blk(il, "ffn_up_exps.weight"));
        const Tensor& de = tt.need(blk(il, "ffn_down_exps.weight"));
        last_route.clear();
        for (auto& r : ranked) {
            last_route.push_back((int32_t)r.first);
            const float weight = r.second / weight_sum;
            const float* gw = ge.deq() + r.first * h * f_exp;  // expert-major contiguous, forward.rs:684-709
            const float* uw = ue.deq() + r.first * h * f_exp;
            const float* dw = de.deq() + r.first * f_exp * h;
            auto gated = mat_vec(gw, h, f_exp, x);
            auto upped = mat_vec(uw, h, f_exp, x);
            std::vector<float> hidden(f_exp);
            for (size_t i = 0; i < f_exp; ++i) hidden[i] = silu(gated[i]) * upped[i];
            auto eo = mat_vec(dw, f_exp, h, hidden.data());
            for (size_t i = 0; i < h; ++i) out[i] += weight * eo[i];
        }
        const float* sgw = tt.need(blk(il, "ffn_gate_inp_shexp.weight")).deq();
        float dot = 0.f;
        for (size_t i = 0; i < h; ++i) dot += x[i] * sgw[i];
        const float sg = sigmoid(dot);
        auto sgated = mat_vec(tt.need(blk(il, "ffn_gate_shexp.weight")).deq(), h, f_sh, x);
        auto supped = mat_vec(tt.need(blk(il, "ffn_up_shexp.weight")).deq(), h, f_sh, x);
        std::vector<float> sh(f_sh);
        for (size_t i = 0; i < f_sh; ++i) sh[i] = silu(sgated[i]) * supped[i];
        auto so = mat_vec(tt.need(blk(il, "ffn_down_shexp.weight")).deq(), f_sh, h, sh.data());
        for (size_t i = 0; i < h; ++i) out[i] += sg * so[i];
        return out;
    }

    // forward.rs:834-932
    std::vector<float> attn_step(uint32_t il, const float* x, uint32_t position, State& st) const {
        const size_t h = arch.hidden_size, hd = arch.attn_head_dim, n_q = arch.n_q_heads, n_kv = arch.n_kv_heads;
        const size_t n_rot = (size_t)((float)hd * arch.partial_rotary_factor);
        auto q_full = mat_vec(tt.need(blk(il, "attn_q.weight")).deq(), h, 2 * n_q * hd, x);
        std::vector<float> qcur(n_q * hd), gate(n_q * hd);
        for (size_t hi = 0; hi < n_q; ++hi) {
            std::copy_n(&q_full[hi * 2 * hd], hd, &qcur[hi * hd]);
            std::copy_n(&q_full[hi * 2 * hd + hd], hd, &gate[hi * hd]);
        }
        const float* qn = tt.need(blk(il, "attn_q_norm.weight")).deq();
        for (size_t hi = 0; hi < n_q; ++hi) {
            auto n = rms_norm(&qcur[hi * hd], hd, qn, RMS_EPS);
            std::copy(n.begin(), n.end(), &qcur[hi * hd]);
        }
        auto kcur = mat_vec(tt.need(blk(il, "attn_k.weight")).deq(), h, n_kv * hd, x);
        auto vcur = mat_vec(tt.need(blk(il, "attn_v.weight")).deq(), h, n_kv * hd, x);
        const float* kn = tt.need(blk(il, "attn_k_norm.weight")).deq();
        for (size_t hi = 0; hi < n_kv; ++hi) {
            auto n = rms_norm(&kcur[hi * hd], hd, kn, RMS_EPS);
            std::copy(n.begin(), n.end(), &kcur[hi * hd]);
        }
        rope_in_place(qcur.data(), n_q, hd, n_rot, position, arch.rope_theta);
        rope_in_place(kcur.data(), n_kv, hd, n_rot, position, arch.rope_theta);
        // KvCache::append (forward.rs:1211-1239): strict monotonic
        if (position != st.n_pos[il]) throw std::runtime_error("oracle: out-of-order kv append");
        if (position >= st.capacity) throw std::runtime_error("oracle: kv capacity exceeded");
        if (st.kv_f16) {
            for (auto& e : kcur) e = f16_to_f32(f32_to_f16(e));
            for (auto& e : vcur) e = f16_to_f32(f32_to_f16(e));
        }
        const size_t stride = n_kv * hd;
        st.k[il].resize((size_t)position * stride);
        st.v[il].resize((size_t)position * stride);
        st.k[il].insert(st.k[il].end(), kcur.begin(), kcur.end());
        st.v[il].insert(st.v[il].end(), vcur.begin(), vcur.end());
        st.n_pos[il] = position + 1;

        const size_t group = n_q / n_kv;
        const float scale = 1.0f / std::sqrt((float)hd);
        const size_t n_pos = st.n_pos[il];
        std::vector<float> attn_out(n_q * hd, 0.f);
#pragma omp parallel for schedule(static) if (n_pos > 256)
        for (long qh = 0; qh < (long)n_q; ++qh) {
            const size_t kvh = (size_t)qh / group;
            const float* qs = &qcur[qh * hd];
            std::vector<float> scores(n_pos);
            for (size_t p = 0; p < n_pos; ++p) {
                const float* ks = &st.k[il][p * stride + kvh * hd];
                float s = 0.f;
                for (size_t i = 0; i < hd; ++i) s += qs[i] * ks[i];
                scores[p] = s * scale;
            }
            softmax_in_place(scores.data(), n_pos);
            float* o = &attn_out[qh * hd];
            for (size_t p = 0; p < n_pos; ++p) {
                const float* vs = &st.v[il][p * stride + kvh * hd];
                const float w = scores[p];
                for (size_t i = 0; i < hd; ++i) o[i] += w * vs[i];
            }
        }
        for (size_t i = 0; i < attn_out.size(); ++i) attn_out[i] *= sigmoid(gate[i]);
        return mat_vec(tt.need(blk(il, "attn_output.weight")).deq(), n_q * hd, h, attn_out.data());
    }

    // forward.rs:940-1107
    std::vector<float> gdn_step(uint32_t il, const float* x, std::vector<float>& conv, std::vector<float>& ssm) const {
        const size_t h = arch.hidden_size, n_v = arch.gdn_n_v_heads, n_k = arch.gdn_n_k_heads, hd = arch.gdn_head_dim;
        const size_t conv_dim = 2 * n_k * hd + n_v * hd, ck = arch.gdn_conv_kernel;
        auto qkv = mat_vec(tt.need(blk(il, "attn_qkv.weight")).deq(), h, conv_dim, x);
        auto z = mat_vec(tt.need(blk(il, "attn_gate.weight")).deq(), h, n_v * hd, x);
        auto beta = mat_vec(tt.need(blk(il, "ssm_beta.weight")).deq(), h, n_v, x);
        for (auto& b : beta) b = sigmoid(b);
        auto alpha = mat_vec(tt.need(blk(il, "ssm_alpha.weight")).deq(), h, n_v, x);
        const float* dt = tt.need(blk(il, "ssm_dt.bias")).deq();
        for (size_t i = 0; i < n_v; ++i) alpha[i] += dt[i];
        const float* a_log = tt.need(blk(il, "ssm_a")).deq();
        std::vector<float> g(n_v);
        for (size_t i = 0; i < n_v; ++i) g[i] = softplus(alpha[i]) * a_log[i];

        const float* conv_w = tt.need(blk(il, "ssm_conv1d.weight")).deq();  // [kernel, conv_dim], kernel fastest
        const size_t kmin1 = ck - 1;
        std::vector<float> conv_out(conv_dim);
        for (size_t c = 0; c < conv_dim; ++c) {
            float s = 0.f;
            for (size_t k = 0; k < ck; ++k) {
                const float xv = k < kmin1 ? conv[k * conv_dim + c] : qkv[c];
                s += conv_w[c * ck + k] * xv;
            }
            conv_out[c] = silu(s);
        }
        for (size_t t = 0; t + 1 < kmin1; ++t)
            for (size_t i = 0; i < conv_dim; ++i) conv[t * conv_dim + i] = conv[(t + 1) * conv_dim + i];
        std::copy(qkv.begin(), qkv.end(), conv.begin() + (kmin1 - 1) * conv_dim);

        std::vector<float> q_full(conv_out.begin(), conv_out.begin() + n_k * hd);
        std::vector<float> k_full(conv_out.begin() + n_k * hd, conv_out.begin() + 2 * n_k * hd);
        const float* v_full = conv_out.data() + 2 * n_k * hd;
        for (size_t hi = 0; hi < n_k; ++hi) {
            l2_norm_in_place(&q_full[hi * hd], hd, RMS_EPS);
            l2_norm_in_place(&k_full[hi * hd], hd, RMS_EPS);
        }
        std::vector<float> o(n_v * hd);
        for (size_t hi = 0; hi < n_v; ++hi) {
            const size_t s_off = hi * hd * hd, hk = hi % n_k;
            const float* q_h = &q_full[hk * hd];
            const float* k_h = &k_full[hk * hd];
            const float* v_h = &v_full[hi * hd];
            const float g_h = std::exp(g[hi]);
            const float b_h = beta[hi];
            std::vector<float> sk(hd);
            for (size_t dv = 0; dv < hd; ++dv) {
                float s = 0.f;
                for (size_t dk = 0; dk < hd; ++dk) s += ssm[s_off + dv * hd + dk] * k_h[dk];
                sk[dv] = s;
            }
            for (size_t dv = 0; dv < hd; ++dv) {
                const float coeff = b_h * (v_h[dv] - g_h * sk[dv]);
                for (size_t dk = 0; dk < hd; ++dk) {
                    const size_t idx = s_off + dv * hd + dk;
                    ssm[idx] = g_h * ssm[idx] + coeff * k_h[dk];
                }
            }
            for (size_t dv = 0; dv < hd; ++dv) {
                float s = 0.f;
                for (size_t dk = 0; dk < hd; ++dk) s += ssm[s_off + dv * hd + dk] * q_h[dk];
                o[hi * hd + dv] = s;
            }
        }
        const float* norm_w = tt.need(blk(il, "ssm_norm.weight")).deq();
        std::vector<float> gated(n_v * hd);
        for (size_t hi = 0; hi < n_v; ++hi) {
            auto n = rms_norm(&o[hi * hd], hd, norm_w, RMS_EPS * (float)hd);
            for (size_t i = 0; i < hd; ++i) gated[hi * hd + i] = n[i] * silu(z[hi * hd + i]);
        }
        return mat_vec(tt.need(blk(il, "ssm_out.weight")).deq(), n_v * hd, h, gated.data());
    }

    // forward.rs:96-163 + :173-220 merged: logits (optional) and captured layers (optional)
    void single_token(int32_t token, uint32_t position, State& st, const uint32_t* layer_ids, size_t n_ids,
                      float* captured /* [n_ids*H] or null */, float* logits /* [V] or null */,
                      float* hidden_pre_norm /* [H] or null */) const {
        if (token < 0 || (uint32_t)token >= arch.vocab_size) throw std::runtime_error("oracle: bad token");
        const size_t h = arch.hidden_size;
        auto x = embed_token(token);
        size_t gdn_idx = 0;
        for (uint32_t il = 0; il < arch.n_layer; ++il) {
            auto cur = rms_norm(x.data(), h, tt.need(blk(il, "attn_norm.weight")).deq(), RMS_EPS);
            std::vector<float> mix;
            if (is_attn(il)) mix = attn_step(il, cur.data(), position, st);
            else { mix = gdn_step(il, cur.data(), st.conv[gdn_idx], st.ssm[gdn_idx]); ++gdn_idx; }
            for (size_t i = 0; i < h; ++i) x[i] += mix[i];
            auto post = rms_norm(x.data(), h, tt.need(blk(il, "post_attention_norm.weight")).deq(), RMS_EPS);
            auto f = ffn(il, post.data());
            for (size_t i = 0; i < h; ++i) x[i] += f[i];
            if (captured)
                for (size_t k = 0; k < n_ids; ++k)
                    if (layer_ids[k] == il) std::copy(x.begin(), x.end(), captured + k * h);
        }
        if (hidden_pre_norm) std::copy(x.begin(), x.end(), hidden_pre_norm);
        if (logits) {
            auto normed = rms_norm(x.data(), h, tt.need("output_norm.weight").deq(), RMS_EPS);
            auto l = mat_vec(lm_head().deq(), h, arch.vocab_size, normed.data());
            std::copy(l.begin(), l.end(), logits);
        }
    }
};

// ---- drafter (forward.rs:380-662) -----------------------------------------
struct Drafter {
    dfl_dflash_config cfg{};
    TensorTable tt;
    std::string blk(uint32_t il, const char* suffix) const { return "blk." + std::to_string(il) + "." + suffix; }

    // returns [N, vocab] logits; hidden_out (optional) receives the [N, H] rows after output_norm, the input of both
    // the lm_head and the DFlash 2 selector's gate projection (metal_dflash.rs:17099-17128)
    std::vector<float> draft(const Model& target, const int32_t* noise_ids, size_t n, const float* target_ctx_stacked,
                             size_t ctx_len, const uint32_t* pos_ctx, uint32_t noise_start_pos, float* hidden_out = nullptr) const {
        const size_t h = cfg.hidden_size, f = cfg.intermediate_size, hd = cfg.head_dim;
        const size_t n_q = cfg.n_q_heads, n_kv = cfg.n_kv_heads, q_dim = n_q * hd, kv_dim = n_kv * hd, group = n_q / n_kv;
        const size_t nfeat = (size_t)cfg.n_target_layers * target.arch.hidden_size;
        const float eps = cfg.rms_norm_eps;
        const float* fc_w = tt.need("dflash_fc.weight").deq();
        const float* hn_w = tt.need("dflash_hidden_norm.weight").deq();
        std::vector<float> ctx_h(h * ctx_len);
        for (size_t c = 0; c < ctx_len; ++c) {
            auto proj = mat_vec(fc_w, nfeat, h, target_ctx_stacked + c * nfeat);
            auto nn = rms_norm(proj.data(), h, hn_w, eps);
            std::copy(nn.begin(), nn.end(), &ctx_h[c * h]);
        }
        std::vector<float> x(n * h);
        for (size_t i = 0; i < n; ++i) {
            if (noise_ids[i] < 0 || (uint32_t)noise_ids[i] >= target.arch.vocab_size) throw std::runtime_error("oracle: bad token");
            auto e = target.embed_token(noise_ids[i]);
            std::copy(e.begin(), e.end(), &x[i * h]);
        }
        const size_t n_rot = hd;
        const float theta = cfg.rope_theta;
        const float kq_scale = 1.0f / std::sqrt((float)hd);
        for (uint32_t il = 0; il < cfg.n_layer; ++il) {
            const float* an = tt.need(blk(il, "attn_norm.weight")).deq();
            std::vector<float> noise_norm(n * h);
            for (size_t i = 0; i < n; ++i) { auto nn = rms_norm(&x[i * h], h, an, eps); std::copy(nn.begin(), nn.end(), &noise_norm[i * h]); }
            const float* q_w = tt.need(blk(il, "attn_q.weight")).deq();
            const float* k_w = tt.need(blk(il, "attn_k.weight")).deq();
            const float* v_w = tt.need(blk(il, "attn_v.weight")).deq();
            std::vector<float> q_full(n * q_dim), k_noise(n * kv_dim), v_noise(n * kv_dim);
            for (size_t i = 0; i < n; ++i) {
                auto r = mat_vec(q_w, h, q_dim, &noise_norm[i * h]); std::copy(r.begin(), r.end(), &q_full[i * q_dim]);
                auto kr = mat_vec(k_w, h, kv_dim, &noise_norm[i * h]); std::copy(kr.begin(), kr.end(), &k_noise[i * kv_dim]);
                auto vr = mat_vec(v_w, h, kv_dim, &noise_norm[i * h]); std::copy(vr.begin(), vr.end(), &v_noise[i * kv_dim]);
            }
            std::vector<float> k_ctx(ctx_len * kv_dim), v_ctx(ctx_len * kv_dim);
            for (size_t c = 0; c < ctx_len; ++c) {
                auto kr = mat_vec(k_w, h, kv_dim, &ctx_h[c * h]); std::copy(kr.begin(), kr.end(), &k_ctx[c * kv_dim]);
                auto vr = mat_vec(v_w, h, kv_dim, &ctx_h[c * h]); std::copy(vr.begin(), vr.end(), &v_ctx[c * kv_dim]);
            }
            const float* qn = tt.need(blk(il, "attn_q_norm.weight")).deq();
            const float* kn = tt.need(blk(il, "attn_k_norm.weight")).deq();
            for (size_t i = 0; i < n; ++i)
                for (size_t hi = 0; hi < n_q; ++hi) { auto nn = rms_norm(&q_full[i * q_dim + hi * hd], hd, qn, eps); std::copy(nn.begin(), nn.end(), &q_full[i * q_dim + hi * hd]); }
            for (size_t i = 0; i < n; ++i)
                for (size_t hi = 0; hi < n_kv; ++hi) { auto nn = rms_norm(&k_noise[i * kv_dim + hi * hd], hd, kn, eps); std::copy(nn.begin(), nn.end(), &k_noise[i * kv_dim + hi * hd]); }
            for (size_t c = 0; c < ctx_len; ++c)
                for (size_t hi = 0; hi < n_kv; ++hi) { auto nn = rms_norm(&k_ctx[c * kv_dim + hi * hd], hd, kn, eps); std::copy(nn.begin(), nn.end(), &k_ctx[c * kv_dim + hi * hd]); }
            for (size_t i = 0; i < n; ++i) {
                rope_in_place(&q_full[i * q_dim], n_q, hd, n_rot, noise_start_pos + (uint32_t)i, theta);
                rope_in_place(&k_noise[i * kv_dim], n_kv, hd, n_rot, noise_start_pos + (uint32_t)i, theta);
            }
            for (size_t c = 0; c < ctx_len; ++c) rope_in_place(&k_ctx[c * kv_dim], n_kv, hd, n_rot, pos_ctx[c], theta);
            const size_t n_tot = ctx_len + n;
            const bool is_swa = cfg.layer_is_swa[il] != 0;
            std::vector<float> attn_out(n * q_dim, 0.f);
            for (size_t qi = 0; qi < n; ++qi) {
                const uint32_t q_pos = noise_start_pos + (uint32_t)qi;
                for (size_t qh = 0; qh < n_q; ++qh) {
                    const size_t kvh = qh / group;
                    const float* qs = &q_full[qi * q_dim + qh * hd];
                    std::vector<float> scores(n_tot, -INFINITY);
                    for (size_t ki = 0; ki < n_tot; ++ki) {
                        const uint32_t k_pos = ki < ctx_len ? pos_ctx[ki] : noise_start_pos + (uint32_t)(ki - ctx_len);
                        const uint32_t diff = q_pos > k_pos ? q_pos - k_pos : k_pos - q_pos;
                        const bool allowed = (!cfg.causal || k_pos <= q_pos) && (!is_swa || cfg.swa_window == 0 || diff < cfg.swa_window);
                        if (!allowed) continue;
                        const float* ks = ki < ctx_len ? &k_ctx[ki * kv_dim + kvh * hd] : &k_noise[(ki - ctx_len) * kv_dim + kvh * hd];
                        float s = 0.f;
                        for (size_t d = 0; d < hd; ++d) s += qs[d] * ks[d];
                        scores[ki] = s * kq_scale;
                    }
                    softmax_in_place(scores.data(), n_tot);
                    float* o = &attn_out[qi * q_dim + qh * hd];
                    for (size_t ki = 0; ki < n_tot; ++ki) {
                        const float w = scores[ki];
                        if (!std::isfinite(w) || w == 0.0f) continue;
                        const float* vs = ki < ctx_len ? &v_ctx[ki * kv_dim + kvh * hd] : &v_noise[(ki - ctx_len) * kv_dim + kvh * hd];
                        for (size_t d = 0; d < hd; ++d) o[d] += w * vs[d];
                    }
                }
            }
            const float* o_w = tt.need(blk(il, "attn_output.weight")).deq();
            for (size_t i = 0; i < n; ++i) {
                auto p = mat_vec(o_w, q_dim, h, &attn_out[i * q_dim]);
                for (size_t j = 0; j < h; ++j) x[i * h + j] += p[j];
            }
            const float* pn = tt.need(blk(il, "post_attention_norm.weight")).deq();
            const float* g_w = tt.need(blk(il, "ffn_gate.weight")).deq();
            const float* u_w = tt.need(blk(il, "ffn_up.weight")).deq();
            const float* d_w = tt.need(blk(il, "ffn_down.weight")).deq();
            for (size_t i = 0; i < n; ++i) {
                auto h2 = rms_norm(&x[i * h], h, pn, eps);
                auto gated = mat_vec(g_w, h, f, h2.data());
                auto upped = mat_vec(u_w, h, f, h2.data());
                std::vector<float> inner(f);
                for (size_t j = 0; j < f; ++j) inner[j] = silu(gated[j]) * upped[j];
                auto down = mat_vec(d_w, f, h, inner.data());
                for (size_t j = 0; j < h; ++j) x[i * h + j] += down[j];
            }
        }
        const float* on_w = tt.need("output_norm.weight").deq();
        const size_t v = target.arch.vocab_size;
        std::vector<float> logits(n * v);
        const float* lm = target.lm_head().deq();
        for (size_t i = 0; i < n; ++i) {
            auto normed = rms_norm(&x[i * h], h, on_w, eps);
            if (hidden_out) std::copy(normed.begin(), normed.end(), hidden_out + i * h);
            auto row = mat_vec(lm, h, v, normed.data());
            std::copy(row.begin(), row.end(), &logits[i * v]);
        }
        return logits;
    }
};

}  // namespace oracle
