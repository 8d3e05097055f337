// DFlash-2 path selector, host side (reference: crates/qwen-llm/src/metal_dflash.rs - DFlash2Codebook :3163-3340,
// select_draft_path :17176-17251, draft_block_sampled :17268-17415).
//
// The two token codebooks ([rank, V], one rank-wide row per token id) stay in host memory, as in the reference: a
// block's walk touches at most 16 rows per draft position.  The device produces, per block, the top-16 (id, logit)
// pairs of every drafter row and the context gate W_h h; the walk below picks, position by position, the candidate b
// maximising  U(b) + < A(prev) * gate, B(b) >  (A = predecessor codebook row of the previous choice, B = successor
// codebook row of the candidate), greedily or by sampling the 16 scores with the proposal sampler.
#include <cmath>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/dflash_b200.h"

namespace dfl {
dfl_status fail(dfl_status st, const std::string& msg);
}
using dfl::fail;

namespace {
inline float f16_bits_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu, bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {  // subnormal: renormalise
            int e = -1;
            do { ++e; man <<= 1; } while (!(man & 0x400u));
            bits = sign | (uint32_t)(127 - 15 - e) << 23 | (man & 0x3FFu) << 13;
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | man << 13;
    } else {
        bits = sign | (exp + 112u) << 23 | man << 13;
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}
inline uint16_t rd16(const uint8_t* p) { return (uint16_t)(p[0] | p[1] << 8); }

// one Q4_K super-block (144 B -> 256 values): d, dmin f16; 12 B of 6-bit scales / mins; 128 B of nibbles;
// value = d * sc * q - dmin * m, in ggml's order of operations
void q4k_block(const uint8_t* b, float* y) {
    const float d = f16_bits_to_f32(rd16(b)), dmin = f16_bits_to_f32(rd16(b + 2));
    const uint8_t* sc = b + 4;
    const uint8_t* q = b + 16;
    auto scale_min = [&](int j, uint8_t& s, uint8_t& m) {
        if (j < 4) {
            s = sc[j] & 63;
            m = sc[j + 4] & 63;
        } else {
            s = (uint8_t)((sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4));
            m = (uint8_t)((sc[j + 4] >> 4) | ((sc[j] >> 6) << 4));
        }
    };
    for (int j = 0; j < 4; ++j) {
        uint8_t s1, m1, s2, m2;
        scale_min(2 * j, s1, m1);
        scale_min(2 * j + 1, s2, m2);
        const float d1 = d * s1, mm1 = dmin * m1, d2 = d * s2, mm2 = dmin * m2;
        for (int l = 0; l < 32; ++l) y[64 * j + l] = d1 * (float)(q[32 * j + l] & 0xF) - mm1;
        for (int l = 0; l < 32; ++l) y[64 * j + 32 + l] = d2 * (float)(q[32 * j + l] >> 4) - mm2;
    }
}
}  // namespace

struct dfl_codebook {
    std::vector<uint8_t> raw;
    int32_t dtype = 0;
    uint64_t rank = 0, n_rows = 0, row_bytes = 0;

    dfl_status dequant_row(uint64_t row, float* out) const {
        if (row >= n_rows) return fail(DFL_ERR_BAD_TOKEN, "selector codebook row out of range");
        const uint8_t* p = raw.data() + row * row_bytes;
        switch (dtype) {
            case DFL_Q4_K:
                q4k_block(p, out);
                break;
            case DFL_Q8_0:
                for (uint64_t b = 0; b < rank / 32; ++b) {
                    const float d = f16_bits_to_f32(rd16(p + 34 * b));
                    for (int j = 0; j < 32; ++j) out[32 * b + j] = d * (float)(int8_t)p[34 * b + 2 + j];
                }
                break;
            case DFL_F32:
                memcpy(out, p, rank * 4);
                break;
            case DFL_F16:
                for (uint64_t i = 0; i < rank; ++i) out[i] = f16_bits_to_f32(rd16(p + 2 * i));
                break;
            case DFL_BF16:
                for (uint64_t i = 0; i < rank; ++i) {
                    const uint32_t bits = (uint32_t)rd16(p + 2 * i) << 16;
                    memcpy(&out[i], &bits, 4);
                }
                break;
            default:
                return fail(DFL_ERR_UNSUPPORTED, "selector codebook dtype");
        }
        return DFL_OK;
    }
};

namespace {
struct WalkInputs {
    const dfl_codebook *pred, *succ;
    uint32_t top_k, rank, n;
    const int32_t* ids;
    const float *vals, *sel_h;
};
dfl_status check_walk(const WalkInputs& w) {
    if (!w.pred || !w.succ || !w.ids || !w.vals || !w.sel_h) return fail(DFL_ERR_BAD_ARG, "selector walk: null argument");
    if (w.n == 0 || w.top_k == 0) return fail(DFL_ERR_BAD_SHAPE, "selector walk: block size and selector top-k must be nonzero");
    if (w.pred->rank != w.rank || w.succ->rank != w.rank) return fail(DFL_ERR_BAD_SHAPE, "selector codebook output rank mismatch");
    return DFL_OK;
}
// scores of one position's candidates; invalid ids (top-k sentinels) keep -inf and scored[b] = 0
dfl_status score_position(const WalkInputs& w, uint32_t pos, const std::vector<float>& pred_row, std::vector<float>& gate,
                          std::vector<float>& succ_row, float* scores, uint8_t* scored) {
    const float* hrow = w.sel_h + (size_t)pos * w.rank;
    for (uint32_t r = 0; r < w.rank; ++r) gate[r] = pred_row[r] * hrow[r];
    for (uint32_t b = 0; b < w.top_k; ++b) {
        const int32_t cand = w.ids[(size_t)pos * w.top_k + b];
        scores[b] = -INFINITY;
        if (scored) scored[b] = 0;
        if (cand < 0 || (uint64_t)cand >= w.succ->n_rows) continue;
        dfl_status s = w.succ->dequant_row((uint64_t)cand, succ_row.data());
        if (s != DFL_OK) return s;
        float dot = 0.f;
        for (uint32_t r = 0; r < w.rank; ++r) dot += gate[r] * succ_row[r];
        scores[b] = w.vals[(size_t)pos * w.top_k + b] + dot;
        if (scored) scored[b] = 1;
    }
    return DFL_OK;
}
}  // namespace

extern "C" {

// DFlash2Codebook::from_gguf  metal_dflash.rs:3180-3273
dfl_status dfl_codebook_create(int32_t dtype, uint64_t rank, uint64_t n_rows, const void* data, uint64_t n_bytes, dfl_codebook** out) {
    if (!data || !out) return fail(DFL_ERR_BAD_ARG, "codebook_create: null argument");
    *out = nullptr;
    if (rank == 0 || n_rows == 0) return fail(DFL_ERR_BAD_SHAPE, "selector codebook dimensions must be nonzero");
    uint64_t blk_el = 1, blk_bytes = 0;
    switch (dtype) {
        case DFL_Q4_K: blk_el = 256; blk_bytes = 144; break;
        case DFL_Q8_0: blk_el = 32; blk_bytes = 34; break;
        case DFL_F32: blk_bytes = 4; break;
        case DFL_F16:
        case DFL_BF16: blk_bytes = 2; break;
        default: return fail(DFL_ERR_UNSUPPORTED, "selector codebook dtype must be Q4_K/Q8_0/F32/F16/BF16");
    }
    if (rank % blk_el) return fail(DFL_ERR_BAD_SHAPE, "selector codebook rank is not block-aligned");
    if (dtype == DFL_Q4_K && rank != 256) return fail(DFL_ERR_BAD_SHAPE, "Q4_K selector codebook rank must be 256");
    const uint64_t row_bytes = rank / blk_el * blk_bytes;
    if (n_rows > UINT64_MAX / row_bytes) return fail(DFL_ERR_BAD_SHAPE, "selector codebook payload size overflows");
    if (n_bytes != row_bytes * n_rows) return fail(DFL_ERR_BAD_SHAPE, "selector codebook payload size mismatch");
    auto* c = new dfl_codebook();
    c->dtype = dtype;
    c->rank = rank;
    c->n_rows = n_rows;
    c->row_bytes = row_bytes;
    c->raw.assign((const uint8_t*)data, (const uint8_t*)data + n_bytes);
    *out = c;
    return DFL_OK;
}
void dfl_codebook_destroy(dfl_codebook* c) { delete c; }

// DFlash2Codebook::dequant_row  metal_dflash.rs:3275-3340
dfl_status dfl_codebook_dequant_row(const dfl_codebook* c, uint64_t row, float* out, uint64_t n_out) {
    if (!c || !out) return fail(DFL_ERR_BAD_ARG, "codebook_dequant_row: null argument");
    if (n_out != c->rank) return fail(DFL_ERR_BAD_SHAPE, "selector codebook output rank mismatch");
    return c->dequant_row(row, out);
}

// select_draft_path  metal_dflash.rs:17176-17251 (scores / scored as in diagnose_dflash2_selector_walk :3472-3620)
dfl_status dfl_selector_walk(const dfl_codebook* pred, const dfl_codebook* succ, uint32_t top_k, uint32_t rank, int32_t carry, uint32_t n,
                             const int32_t* ids, const float* vals, const float* sel_h, int32_t* tokens_out, float* scores_out,
                             uint8_t* scored_out) {
    const WalkInputs w{pred, succ, top_k, rank, n, ids, vals, sel_h};
    dfl_status s = check_walk(w);
    if (s != DFL_OK) return s;
    if (!tokens_out) return fail(DFL_ERR_BAD_ARG, "selector walk: null argument");
    std::vector<float> pred_row(rank), succ_row(rank), gate(rank), scores(top_k);
    for (uint32_t i = 0; i < n; ++i) tokens_out[i] = ids[0];   // slot 0 = the anchor row's top-1, never read by the driver
    if (carry < 0) return fail(DFL_ERR_BAD_TOKEN, "selector codebook row out of range");
    if ((s = pred->dequant_row((uint64_t)carry, pred_row.data())) != DFL_OK) return s;
    for (uint32_t pos = 1; pos < n; ++pos) {
        uint8_t* scored = scored_out ? scored_out + (size_t)pos * top_k : nullptr;
        if ((s = score_position(w, pos, pred_row, gate, succ_row, scores.data(), scored)) != DFL_OK) return s;
        uint32_t best_b = 0;
        float best = -INFINITY;
        for (uint32_t b = 0; b < top_k; ++b) {
            const int32_t cand = ids[(size_t)pos * top_k + b];
            if (cand < 0 || (uint64_t)cand >= succ->n_rows) continue;
            if (scores[b] > best) {   // strict: first (highest unary rank) candidate wins ties, NaN never wins
                best = scores[b];
                best_b = b;
            }
        }
        if (scores_out) memcpy(scores_out + (size_t)pos * top_k, scores.data(), top_k * 4);
        const int32_t chosen = ids[(size_t)pos * top_k + best_b];
        tokens_out[pos] = chosen;
        if (chosen < 0) return fail(DFL_ERR_BAD_TOKEN, "selector codebook row out of range");
        if ((s = pred->dequant_row((uint64_t)chosen, pred_row.data())) != DFL_OK) return s;
    }
    return DFL_OK;
}

// the walk of draft_block_sampled  metal_dflash.rs:17349-17409; proposals as dfl_sparse_proposals rows 0 .. n-2
dfl_status dfl_selector_walk_sampled(const dfl_codebook* pred, const dfl_codebook* succ, uint32_t top_k, uint32_t rank, int32_t carry,
                                     uint32_t n, const int32_t* ids, const float* vals, const float* sel_h, dfl_sampler* proposal_sampler,
                                     int32_t* tokens_out, uint32_t* cand_offsets, int32_t* cand_tokens, double* cand_weights) {
    const WalkInputs w{pred, succ, top_k, rank, n, ids, vals, sel_h};
    dfl_status s = check_walk(w);
    if (s != DFL_OK) return s;
    if (!proposal_sampler || !tokens_out || !cand_offsets || !cand_tokens || !cand_weights)
        return fail(DFL_ERR_BAD_ARG, "selector walk: null argument");
    dfl_sampling_config pc;
    dfl_sampler_get_config(proposal_sampler, &pc);
    if (!(pc.temperature > 0.0f) || pc.top_k != 0 || pc.top_p != 1.0f || pc.min_p != 0.0f)
        return fail(DFL_ERR_SAMPLING, "DFlash 2 proposal sampler must use temperature without target filters");
    std::vector<float> pred_row(rank), succ_row(rank), gate(rank), scores(top_k);
    std::vector<int32_t> dt(top_k);
    std::vector<double> dw(top_k);
    for (uint32_t i = 0; i < n; ++i) tokens_out[i] = ids[0];
    if (carry < 0) return fail(DFL_ERR_BAD_TOKEN, "selector codebook row out of range");
    if ((s = pred->dequant_row((uint64_t)carry, pred_row.data())) != DFL_OK) return s;
    uint32_t n_cand = 0;
    cand_offsets[0] = 0;
    for (uint32_t pos = 1; pos < n; ++pos) {
        if ((s = score_position(w, pos, pred_row, gate, succ_row, scores.data(), nullptr)) != DFL_OK) return s;
        int32_t sel = 0;
        uint64_t ci = 0, count = 0;
        double total = 0;
        if ((s = dfl_sampler_sample_with_distribution(proposal_sampler, scores.data(), top_k, &sel, &ci, dt.data(), dw.data(), top_k, &count,
                                                      &total)) != DFL_OK)
            return s;
        if (sel < 0 || (uint32_t)sel >= top_k) return fail(DFL_ERR_SAMPLING, "sampled selector candidate index is out of range");
        const int32_t token = ids[(size_t)pos * top_k + sel];
        if (token < 0 || (uint64_t)token >= pred->n_rows) return fail(DFL_ERR_BAD_TOKEN, "sampled selector returned an invalid token");
        for (uint64_t k = 0; k < count && k < top_k; ++k)
            if (dw[k] > 0.0) {
                cand_tokens[n_cand] = ids[(size_t)pos * top_k + dt[k]];
                cand_weights[n_cand] = dw[k];
                ++n_cand;
            }
        cand_offsets[pos] = n_cand;
        tokens_out[pos] = token;
        if ((s = pred->dequant_row((uint64_t)token, pred_row.data())) != DFL_OK) return s;
    }
    return DFL_OK;
}

}  // extern "C"
