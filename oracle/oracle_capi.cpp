// TEST INFRASTRUCTURE — C entry points of the CPU oracle for ctypes.  Only tests,
// the smoke check and the benchmark's CPU-baseline leg load this library; the
// product library never does.
#include <chrono>
#ifdef _OPENMP
#include <omp.h>
#endif
#include <cstdio>
#include <cstring>
#include <string>

#include "forward.hpp"

using namespace oracle;

static thread_local std::string g_err;
#define ORC_TRY try {
#define ORC_CATCH                     \
    }                                 \
    catch (const std::exception& e) { \
        g_err = e.what();             \
        return 1;                     \
    }                                 \
    return 0;

extern "C" {

const char* orc_last_error() { return g_err.c_str(); }

int orc_dequant(int32_t dtype, const uint8_t* src, uint64_t n_elements, float* out) {
    ORC_TRY dequant_to_f32(dtype, src, n_elements, out);
    ORC_CATCH
}
int orc_quantize(int32_t dtype, const float* x, uint64_t n_elements, uint8_t* out) {
    ORC_TRY quantize_from_f32(dtype, x, n_elements, out);
    ORC_CATCH
}
uint64_t orc_storage_bytes(int32_t dtype, uint64_t n_elements) {
    uint64_t blk, bytes;
    try { storage_layout(dtype, blk, bytes); } catch (...) { return 0; }
    if (n_elements % blk) return 0;
    return n_elements / blk * bytes;
}
uint16_t orc_f32_to_f16(float f) { return f32_to_f16(f); }
float orc_f16_to_f32(uint16_t h) { return f16_to_f32(h); }

// y[r][o] = sum_i x[r][i] W[o][i] with the oracle's sequential order.
int orc_matmul(int32_t dtype, const uint8_t* w, uint64_t n_in, uint64_t n_out, const float* x, int32_t n_rows, float* y) {
    ORC_TRY
    std::vector<float> wf(n_in * n_out);
    dequant_to_f32(dtype, w, n_in * n_out, wf.data());
    for (int r = 0; r < n_rows; ++r) {
        auto row = mat_vec(wf.data(), n_in, n_out, x + (size_t)r * n_in);
        std::copy(row.begin(), row.end(), y + (size_t)r * n_out);
    }
    ORC_CATCH
}

// Same product from an already dequantised f32 matrix (used by the timed CPU baseline so that
// dequantisation is not re-done per step).
int orc_matmul_f32(const float* wf, uint64_t n_in, uint64_t n_out, const float* x, int32_t n_rows, float* y) {
    ORC_TRY
    for (int r = 0; r < n_rows; ++r) {
        auto row = mat_vec(wf, n_in, n_out, x + (size_t)r * n_in);
        std::copy(row.begin(), row.end(), y + (size_t)r * n_out);
    }
    ORC_CATCH
}

// greedy_token (sampling.rs:1159-1181): total order, lowest index on ties. Returns -1-index on NaN.
int32_t orc_greedy_token(const float* logits, uint64_t n) {
    auto key = [](float f) { int32_t b; std::memcpy(&b, &f, 4); return b < 0 ? (int32_t)(b ^ 0x7fffffff) : b; };
    if (n == 0) return INT32_MIN;
    if (std::isnan(logits[0])) return -1;
    uint64_t best = 0;
    for (uint64_t i = 1; i < n; ++i) {
        if (std::isnan(logits[i])) return -1 - (int32_t)i;
        if (key(logits[i]) > key(logits[best])) best = i;
    }
    return (int32_t)best;
}

// ---- model / state ------------------------------------------------------
void* orc_model_create(const dfl_arch* arch, const dfl_tensor* tensors, uint64_t n) {
    try {
        auto* m = new Model();
        m->arch = *arch;
        for (uint64_t i = 0; i < n; ++i) m->tt.add(tensors[i]);
        return m;
    } catch (const std::exception& e) { g_err = e.what(); return nullptr; }
}
void orc_model_destroy(void* m) { delete (Model*)m; }
void orc_model_drop_caches(void* m) { for (auto& kv : ((Model*)m)->tt.t) kv.second.drop_cache(); }

void* orc_state_create(void* m, uint64_t kv_capacity, int32_t kv_f16) {
    return new State(((Model*)m)->fresh_state(kv_capacity, kv_f16 != 0));
}
void* orc_state_clone(void* s) { return new State(*(State*)s); }
void orc_state_destroy(void* s) { delete (State*)s; }
uint64_t orc_state_n_pos(void* m, void* s) {
    auto* M = (Model*)m; auto* S = (State*)s;
    for (uint32_t il = 0; il < M->arch.n_layer; ++il) if (M->is_attn(il)) return S->n_pos[il];
    return 0;
}
int orc_state_read_gdn(void* s, uint32_t gdn_index, float* ssm, float* conv) {
    auto* S = (State*)s;
    if (gdn_index >= S->ssm.size()) return 1;
    if (ssm) std::copy(S->ssm[gdn_index].begin(), S->ssm[gdn_index].end(), ssm);
    if (conv) std::copy(S->conv[gdn_index].begin(), S->conv[gdn_index].end(), conv);
    return 0;
}
// K/V row of the attn_index-th attention layer at `pos`.
int orc_state_read_kv(void* m, void* s, uint32_t attn_index, uint32_t pos, float* k, float* v) {
    auto* M = (Model*)m; auto* S = (State*)s;
    uint32_t seen = 0;
    for (uint32_t il = 0; il < M->arch.n_layer; ++il) {
        if (!M->is_attn(il)) continue;
        if (seen++ == attn_index) {
            const size_t stride = (size_t)M->arch.n_kv_heads * M->arch.attn_head_dim;
            if (pos >= S->n_pos[il]) return 1;
            std::copy_n(&S->k[il][pos * stride], stride, k);
            std::copy_n(&S->v[il][pos * stride], stride, v);
            return 0;
        }
    }
    return 1;
}

int orc_single_token(void* m, void* s, int32_t token, uint32_t position, const uint32_t* layer_ids, uint32_t n_ids,
                     float* captured, float* logits, float* hidden) {
    ORC_TRY((Model*)m)->single_token(token, position, *(State*)s, layer_ids, n_ids, captured, logits, hidden);
    ORC_CATCH
}

// Expert ids picked by the last MoE routing call (top-k indices, bit-exact contract).
int orc_last_route(void* m, int32_t* out, uint32_t cap) {
    auto& r = ((Model*)m)->last_route;
    uint32_t n = (uint32_t)std::min<size_t>(cap, r.size());
    std::copy_n(r.begin(), n, out);
    return (int)n;
}

// One FFN / MoE call on a given layer (unit-level parity for routing).
int orc_ffn(void* m, uint32_t il, const float* x, float* out) {
    ORC_TRY
    auto y = ((Model*)m)->ffn(il, x);
    std::copy(y.begin(), y.end(), out);
    ORC_CATCH
}

void* orc_drafter_create(const dfl_dflash_config* cfg, const dfl_tensor* tensors, uint64_t n) {
    try {
        auto* d = new Drafter();
        d->cfg = *cfg;
        for (uint64_t i = 0; i < n; ++i) d->tt.add(tensors[i]);
        return d;
    } catch (const std::exception& e) { g_err = e.what(); return nullptr; }
}
void orc_drafter_destroy(void* d) { delete (Drafter*)d; }

int orc_dflash_draft(void* drafter, void* target, const int32_t* noise_ids, uint32_t n, const float* ctx_stacked,
                     uint32_t ctx_len, const uint32_t* pos_ctx, uint32_t noise_start_pos, float* logits_out) {
    ORC_TRY
    auto l = ((Drafter*)drafter)->draft(*(Model*)target, noise_ids, n, ctx_stacked, ctx_len, pos_ctx, noise_start_pos);
    std::copy(l.begin(), l.end(), logits_out);
    ORC_CATCH
}

// the same pass, also returning the normalised final hidden rows [n][H]
int orc_dflash_draft_hidden(void* drafter, void* target, const int32_t* noise_ids, uint32_t n, const float* ctx_stacked,
                            uint32_t ctx_len, const uint32_t* pos_ctx, uint32_t noise_start_pos, float* logits_out, float* hidden_out) {
    ORC_TRY
    auto l = ((Drafter*)drafter)->draft(*(Model*)target, noise_ids, n, ctx_stacked, ctx_len, pos_ctx, noise_start_pos, hidden_out);
    std::copy(l.begin(), l.end(), logits_out);
    ORC_CATCH
}

int orc_num_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// The scalar primitives on their own (forward.rs:1256-1309), for the reference's known-answer checks (forward.rs:1377-1414).
// kind: 0 rms_norm(x, w, eps) -> out, 1 l2_norm_in_place(eps), 2 softmax_in_place, 3 silu, 4 softplus, 5 sigmoid (element-wise).
int orc_primitive(int32_t kind, const float* x, uint64_t n, const float* w, float eps, float* out) {
    ORC_TRY
    switch (kind) {
        case 0: { auto y = rms_norm(x, n, w, eps); std::copy(y.begin(), y.end(), out); break; }
        case 1: std::copy(x, x + n, out); l2_norm_in_place(out, n, eps); break;
        case 2: std::copy(x, x + n, out); softmax_in_place(out, n); break;
        case 3: for (uint64_t i = 0; i < n; ++i) out[i] = silu(x[i]); break;
        case 4: for (uint64_t i = 0; i < n; ++i) out[i] = softplus(x[i]); break;
        case 5: for (uint64_t i = 0; i < n; ++i) out[i] = sigmoid(x[i]); break;
        default: throw std::runtime_error("oracle: unknown primitive");
    }
    ORC_CATCH
}

// Sets the number of OpenMP threads the timed CPU baseline uses (a launcher may have exported OMP_NUM_THREADS=1);
// returns the count in effect.
int orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
    return omp_get_max_threads();
#else
    (void)n;
    return 1;
#endif
}

}  // extern "C"
