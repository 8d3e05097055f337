// Host-side sampler and DFlash accept-prefix decision (f64, version-1 semantics).
// Product implementation of crates/qwen-llm/src/sampling.rs (`Sampler::{new, at_draw, sample,
// diagnose, couple_deterministic_proposal, couple_sparse_proposal}` :340-790, `greedy_token`
// :1159-1181, candidate keys :1206-1235, radix order :1283-1339, weights / top-p / categorical
// :1370-1438, xoshiro256++ / SplitMix64 :1619-1670) and crates/qwen-llm/src/metal_dflash/accept.rs
// (`decide_dflash_accept_prefix` :76-183).  Acceptance runs on the host in the reference too.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstring>
#include <thread>
#include <limits>
#include <string>
#include <vector>

#include "../../include/dflash_b200.h"

namespace dfl {
dfl_status fail(dfl_status st, const std::string& msg);
}
using dfl::fail;

namespace {

struct SplitMix64 {
    uint64_t s;
    uint64_t next() {
        s += 0x9e3779b97f4a7c15ull;
        uint64_t v = s;
        v = (v ^ (v >> 30)) * 0xbf58476d1ce4e5b9ull;
        v = (v ^ (v >> 27)) * 0x94d049bb133111ebull;
        return v ^ (v >> 31);
    }
};
inline uint64_t rotl(uint64_t x, int k) { return (x << k) | (x >> (64 - k)); }
struct Xoshiro {
    uint64_t st[4];
    void seed(uint64_t seed) {
        SplitMix64 sm{seed};
        for (auto& v : st) v = sm.next();
    }
    uint64_t next_u64() {
        const uint64_t result = rotl(st[0] + st[3], 23) + st[0];
        const uint64_t t = st[1] << 17;
        st[2] ^= st[0];
        st[3] ^= st[1];
        st[1] ^= st[2];
        st[0] ^= st[3];
        st[2] ^= t;
        st[3] = rotl(st[3], 45);
        return result;
    }
    double next_unit() { return (double)(next_u64() >> 11) / 9007199254740992.0; }
};

enum SErr { S_OK = 0, S_EMPTY, S_NAN, S_TOO_LARGE, S_NO_CANDIDATES, S_PROPOSAL_RANGE, S_PROPOSAL_WEIGHT, S_MISSING_PROPOSAL };

// ascending u32 order == descending f32 total order
inline uint32_t descending_bits(float f) {
    uint32_t b;
    std::memcpy(&b, &f, 4);
    const uint32_t asc = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
    return ~asc;
}
inline double key_logit(uint64_t key) {
    const uint32_t asc = ~(uint32_t)(key >> 32);
    const uint32_t bits = (asc & 0x80000000u) ? (asc & 0x7fffffffu) : ~asc;
    float f;
    std::memcpy(&f, &bits, 4);
    return (double)f;
}
inline int32_t key_token(uint64_t key) { return (int32_t)(uint32_t)key; }

struct Buffers {
    std::vector<uint64_t> keys, scratch;
    std::vector<double> cumulative;
};

// Keys of a row from an order made elsewhere (the device): token order[i] is the i-th candidate.  The order is checked
// - every token in range, keys non-decreasing, which for a permutation is exactly "sorted, ties by ascending token"
// when equal keys also ascend in token - and refused (false) when it is not this row's order.
bool keys_from_order(const float* logits, uint64_t n, const uint32_t* order, uint64_t take, std::vector<uint64_t>& keys) {
    keys.resize(take);
    uint64_t prev = 0;
    for (uint64_t i = 0; i < take; ++i) {
        const uint32_t t = order[i];
        if (t >= n) return false;
        const uint64_t k = ((uint64_t)descending_bits(logits[t]) << 32) | t;
        if (i && k <= prev) return false;   // strictly increasing 64-bit keys: sorted by logit, then by token, no repeats
        keys[i] = k;
        prev = k;
    }
    return true;
}

// Orders candidate keys: whole row when top-k is off, else the top_k best.  Returns count or error.
SErr order_keys(const float* logits, uint64_t n, uint64_t top_k, Buffers& b, uint64_t* count, uint64_t* nan_token,
                const uint32_t* order = nullptr, bool* order_used = nullptr) {
    if (n == 0) return S_EMPTY;
    if (n > 0x7fffffffull) return S_TOO_LARGE;
    const bool full = top_k == 0 || top_k >= n;
    if (order) {
        for (uint64_t t = 0; t < n; ++t)
            if (std::isnan(logits[t])) { *nan_token = t; return S_NAN; }
        const uint64_t take = full ? n : top_k;
        // a prefix of a sorted permutation is the sorted top-k; for the whole row the strict increase over n keys in
        // [0, n) token range makes it a permutation
        if (keys_from_order(logits, n, order, take, b.keys)) {
            *count = take;
            if (order_used) *order_used = true;
            return S_OK;
        }
    }
    b.keys.resize(n);
    // keys in token order; the four byte histograms of the logit half are taken in the same pass
    uint32_t hist[4][256];
    if (full) std::memset(hist, 0, sizeof(hist));
    for (uint64_t t = 0; t < n; ++t) {
        if (std::isnan(logits[t])) { *nan_token = t; return S_NAN; }
        const uint32_t d = descending_bits(logits[t]);
        b.keys[t] = ((uint64_t)d << 32) | t;
        if (full) { ++hist[0][d & 255]; ++hist[1][(d >> 8) & 255]; ++hist[2][(d >> 16) & 255]; ++hist[3][d >> 24]; }
    }
    if (full) {
        // stable LSD radix over the logit half, one byte per pass (256 write streams stay in the first-level cache);
        // keys were built in token order, so equal logits keep ascending token order
        if (n >= 2) {
            b.scratch.resize(n);
            for (int digit = 0; digit < 4; ++digit) {
                const int shift = 32 + 8 * digit;
                uint32_t* h = hist[digit];
                if (h[(b.keys[0] >> shift) & 255] == n) continue;   // every key has the same byte here
                uint32_t off = 0;
                for (int i = 0; i < 256; ++i) { const uint32_t c = h[i]; h[i] = off; off += c; }
                const uint64_t* src = b.keys.data();
                uint64_t* dst = b.scratch.data();
                for (uint64_t i = 0; i < n; ++i) dst[h[(src[i] >> shift) & 255]++] = src[i];
                b.keys.swap(b.scratch);
            }
        }
        *count = n;
    } else {
        std::nth_element(b.keys.begin(), b.keys.begin() + top_k, b.keys.end());
        std::sort(b.keys.begin(), b.keys.begin() + top_k);
        *count = top_k;
    }
    return S_OK;
}

struct Dist {
    std::vector<int32_t> tokens;
    std::vector<double> weights;
    double total = 0;
    int32_t sampled = 0;
    uint64_t index = 0;
};

}  // namespace

struct dfl_sampler {
    dfl_sampling_config cfg;
    Xoshiro rng;
    uint64_t draws = 0;
    Buffers buf;
    // Distributions of a block's rows built ahead of the sequential accept loop, one host thread per row: building a
    // row's distribution draws nothing from the generator, so only the picks have to stay in row order.  Rows are
    // built in waves as the loop reaches them (the first wave covers a typical accepted prefix), so a block rejected
    // early does not pay for all of its rows.
    struct Prepared {
        const float* logits = nullptr;
        Dist dist;
        SErr err = S_OK;
        uint64_t nan_token = 0;
        Buffers buf;
    };
    // rows whose order was made elsewhere (dfl_sampler_set_row_order)
    const float* ord_logits = nullptr;
    const uint32_t* ord_base = nullptr;
    uint32_t ord_rows = 0;
    uint64_t ord_vocab = 0;
    mutable std::atomic<uint64_t> ord_used{0};   // rows that took a registered order (rows are built on several threads)
    uint32_t workers = 0;   // threads that build a block's rows ahead of the accept loop: 0 = the host's concurrency, 1 = none
    const uint32_t* order_for(const float* logits, uint64_t n) const {
        if (!ord_logits || n != ord_vocab || logits < ord_logits) return nullptr;
        const uint64_t off = (uint64_t)(logits - ord_logits);
        if (off % ord_vocab || off / ord_vocab >= ord_rows) return nullptr;
        return ord_base + off;
    }
    std::vector<Prepared> prepared;
    const float* block_logits = nullptr;
    uint64_t block_vocab = 0;
    uint32_t block_rows = 0, n_prepared = 0;

    void prepare_rows(const float* logits, uint32_t n_rows, uint64_t vocab) {
        block_logits = nullptr;
        n_prepared = block_rows = 0;
        if (cfg.temperature == 0.0f || n_rows < 2 || vocab < 4096 || worker_limit() < 2) return;
        block_logits = logits;
        block_vocab = vocab;
        block_rows = n_rows;
        if (prepared.size() < n_rows) prepared.resize(n_rows);
    }
    void end_block() { block_logits = nullptr; n_prepared = block_rows = 0; }
    unsigned worker_limit() const { return workers ? workers : std::thread::hardware_concurrency(); }
    void prepare_wave(uint32_t upto) {
        const unsigned hw = std::max(2u, worker_limit());
        const uint32_t first = n_prepared, last = std::min(block_rows, std::max(upto + 1, first + std::min<uint32_t>(hw, first == 0 ? 6 : 10)));
        const uint32_t n_threads = std::min<uint32_t>(last - first, hw);
        auto work = [&](uint32_t t) {
            for (uint32_t r = first + t; r < last; r += n_threads) {
                Prepared& p = prepared[r];
                p.logits = block_logits + (uint64_t)r * block_vocab;
                p.err = distribution(p.logits, block_vocab, p.dist, &p.nan_token, p.buf);
            }
        };
        std::vector<std::thread> pool;
        for (uint32_t t = 1; t < n_threads; ++t) pool.emplace_back(work, t);
        work(0);
        for (auto& t : pool) t.join();
        n_prepared = last;
    }
    // the prepared distribution of this row, if it belongs to the current block (moved out: a row is consumed once)
    bool take_prepared(const float* logits, Dist& d, SErr* e, uint64_t* nan_token) {
        if (!block_logits || logits < block_logits) return false;
        const uint64_t off = (uint64_t)(logits - block_logits);
        if (off % block_vocab || off / block_vocab >= block_rows) return false;
        const uint32_t r = (uint32_t)(off / block_vocab);
        if (r >= n_prepared) prepare_wave(r);
        if (prepared[r].logits != logits) return false;
        *e = prepared[r].err;
        *nan_token = prepared[r].nan_token;
        std::swap(d, prepared[r].dist);
        prepared[r].logits = nullptr;
        return true;
    }

    // The filtered categorical distribution of sampler-v1 (diagnose_candidates, sampling.rs:1541-1614).
    SErr distribution(const float* logits, uint64_t n, Dist& d, uint64_t* nan_token) {
        SErr e;
        if (take_prepared(logits, d, &e, nan_token)) return e;
        return distribution(logits, n, d, nan_token, buf);
    }
    SErr distribution(const float* logits, uint64_t n, Dist& d, uint64_t* nan_token, Buffers& buf) const {
        uint64_t len = 0;
        bool order_used = false;
        SErr e = order_keys(logits, n, cfg.top_k, buf, &len, nan_token, order_for(logits, n), &order_used);
        if (order_used) ord_used.fetch_add(1, std::memory_order_relaxed);
        if (e != S_OK) return e;
        const uint64_t* keys = buf.keys.data();
        if (cfg.min_p > 0.0f) {
            const double max_logit = key_logit(keys[0]);
            if (std::isfinite(max_logit)) {
                const double threshold = max_logit + std::log((double)cfg.min_p);
                uint64_t keep = 0;
                while (keep < len && key_logit(keys[keep]) >= threshold) ++keep;  // monotone along the order
                len = keep;
            }
        }
        if (len == 0) return S_NO_CANDIDATES;
        const double inf = std::numeric_limits<double>::infinity();
        if (key_logit(keys[0]) == inf) {
            uint64_t keep = 0;
            while (keep < len && key_logit(keys[keep]) == inf) ++keep;
            len = keep;
        }
        d.tokens.resize(len);
        d.weights.resize(len);
        const double t = (double)cfg.temperature;
        if (key_logit(keys[0]) == inf) {
            for (uint64_t i = 0; i < len; ++i) d.weights[i] = 1.0;
        } else {
            const double max_logit = key_logit(keys[0]) / t;
            if (max_logit == -inf) return S_NO_CANDIDATES;
            bool finite = true;
            double* w = d.weights.data();
            for (uint64_t i = 0; i < len; ++i) w[i] = key_logit(keys[i]) / t - max_logit;   // vectorisable part first
            for (uint64_t i = 0; i < len; ++i) {
                w[i] = std::exp(w[i]);
                finite &= std::isfinite(w[i]);
            }
            if (!finite) return S_NO_CANDIDATES;
        }
        for (uint64_t i = 0; i < len; ++i) d.tokens[i] = key_token(keys[i]);
        if (cfg.top_p < 1.0f) {
            double total = 0.0;
            for (uint64_t i = 0; i < len; ++i) total += d.weights[i];
            const double target = total * (double)cfg.top_p;
            double cum = 0.0;
            uint64_t keep = 0;
            for (uint64_t i = 0; i < len; ++i) {
                cum += d.weights[i];
                ++keep;
                if (cum >= target) break;
            }
            keep = std::max<uint64_t>(keep, 1);
            d.tokens.resize(keep);
            d.weights.resize(keep);
        }
        double total = 0.0;
        for (double w : d.weights) total += w;
        if (!(std::isfinite(total) && total > 0.0)) return S_NO_CANDIDATES;
        d.total = total;
        return S_OK;
    }

    static void pick(Dist& d, double uniform) {
        const double target = uniform * d.total;
        double cum = 0.0;
        uint64_t idx = d.weights.size() - 1;
        for (uint64_t i = 0; i < d.weights.size(); ++i) {
            cum += d.weights[i];
            if (target < cum) { idx = i; break; }
        }
        d.index = idx;
        d.sampled = d.tokens[idx];
    }

    static SErr greedy(const float* logits, uint64_t n, int32_t* tok, uint64_t* nan_token) {
        if (n == 0) return S_EMPTY;
        if (n > 0x7fffffffull) return S_TOO_LARGE;
        if (std::isnan(logits[0])) { *nan_token = 0; return S_NAN; }
        uint64_t best = 0;
        uint32_t best_key = descending_bits(logits[0]);
        for (uint64_t t = 1; t < n; ++t) {
            if (std::isnan(logits[t])) { *nan_token = t; return S_NAN; }
            const uint32_t k = descending_bits(logits[t]);
            if (k < best_key) { best = t; best_key = k; }  // strictly greater in total order: lowest index wins ties
        }
        *tok = (int32_t)best;
        return S_OK;
    }

    // Sampler::diagnose with uniform 0 (used by the sparse coupling)
    SErr diagnose0(const float* logits, uint64_t n, Dist& d, uint64_t* nan_token) {
        if (cfg.temperature == 0.0f) {
            int32_t tok;
            SErr e = greedy(logits, n, &tok, nan_token);
            if (e != S_OK) return e;
            d.tokens.assign(1, tok);
            d.weights.assign(1, 1.0);
            d.total = 1.0;
            d.sampled = tok;
            d.index = 0;
            return S_OK;
        }
        SErr e = distribution(logits, n, d, nan_token);
        if (e != S_OK) return e;
        pick(d, 0.0);
        return S_OK;
    }

    SErr sample(const float* logits, uint64_t n, int32_t* tok, uint64_t* idx, uint64_t* nan_token) {
        if (cfg.temperature == 0.0f) {
            *idx = 0;
            return greedy(logits, n, tok, nan_token);
        }
        Dist d;
        SErr e = distribution(logits, n, d, nan_token);
        if (e != S_OK) return e;
        ++draws;
        pick(d, rng.next_unit());
        *tok = d.sampled;
        *idx = d.index;
        return S_OK;
    }

    // returns accepted flag; on rejection *correction is the residual draw (sampling.rs:708-790)
    SErr couple_sparse(const float* logits, uint64_t n, int32_t ptoken, const int32_t* ctok, const double* cw, uint32_t nc, bool* accepted,
                       int32_t* correction, uint64_t* nan_token) {
        if (ptoken < 0 || (uint64_t)ptoken >= n) return S_PROPOSAL_RANGE;
        if (nc == 0) return S_NO_CANDIDATES;
        double ptotal = 0.0, pw = 0.0;
        for (uint32_t i = 0; i < nc; ++i) {
            if (ctok[i] < 0 || (uint64_t)ctok[i] >= n) return S_PROPOSAL_RANGE;
            if (!std::isfinite(cw[i]) || cw[i] < 0.0) return S_PROPOSAL_WEIGHT;
            ptotal += cw[i];
            if (ctok[i] == ptoken) pw += cw[i];
        }
        if (!(std::isfinite(ptotal) && ptotal > 0.0)) return S_NO_CANDIDATES;
        if (!(std::isfinite(pw) && pw > 0.0)) return S_MISSING_PROPOSAL;
        Dist d;
        SErr e = diagnose0(logits, n, d, nan_token);
        if (e != S_OK) return e;
        double tsum = 0.0;
        for (size_t i = 0; i < d.tokens.size(); ++i)
            if (d.tokens[i] == ptoken) tsum += d.weights[i];
        const double tp = tsum / d.total;
        const double pp = pw / ptotal;
        const double acc = std::min(tp / pp, 1.0);
        ++draws;
        if (rng.next_unit() < acc) { *accepted = true; return S_OK; }
        std::vector<double> residual(d.tokens.size());
        double rtotal = 0.0;
        for (size_t i = 0; i < d.tokens.size(); ++i) {
            const double tpi = d.weights[i] / d.total;
            double ps = 0.0;
            for (uint32_t j = 0; j < nc; ++j)
                if (ctok[j] == d.tokens[i]) ps += cw[j];
            const double w = std::max(tpi - ps / ptotal, 0.0);
            rtotal += w;
            residual[i] = w;
        }
        if (!(std::isfinite(rtotal) && rtotal > 0.0)) return S_NO_CANDIDATES;
        ++draws;
        const double threshold = rng.next_unit() * rtotal;
        double cum = 0.0;
        *accepted = false;
        for (size_t i = 0; i < residual.size(); ++i) {
            cum += residual[i];
            if (threshold < cum) { *correction = d.tokens[i]; return S_OK; }
        }
        *correction = d.tokens.back();
        return S_OK;
    }
};

namespace {
dfl_status sampling_fail(SErr e, uint64_t nan_token, int row) {
    const std::string where = row >= 0 ? "DFlash target row " + std::to_string(row) + ": " : "";
    switch (e) {
        case S_EMPTY: return fail(DFL_ERR_SAMPLING, where + "sampling requires a non-empty logits row");
        case S_NAN: return fail(DFL_ERR_SAMPLING, where + "logit at token " + std::to_string(nan_token) + " is NaN");
        case S_TOO_LARGE: return fail(DFL_ERR_SAMPLING, where + "vocabulary size exceeds i32 token ids");
        case S_NO_CANDIDATES: return fail(DFL_ERR_SAMPLING, where + "sampling retained no finite-probability candidates");
        case S_PROPOSAL_RANGE: return fail(DFL_ERR_SAMPLING, where + "proposal token is outside the target vocabulary");
        case S_PROPOSAL_WEIGHT: return fail(DFL_ERR_SAMPLING, where + "proposal weight must be finite and non-negative");
        case S_MISSING_PROPOSAL: return fail(DFL_ERR_SAMPLING, where + "sampled proposal token has no positive proposal weight");
        default: return DFL_OK;
    }
}
bool valid_config(const dfl_sampling_config& c, std::string* why) {
    if (!std::isfinite(c.temperature) || c.temperature < 0.0f) { *why = "sampling temperature must be finite and >= 0"; return false; }
    if (!std::isfinite(c.top_p) || !(0.0f < c.top_p && c.top_p <= 1.0f)) { *why = "top_p must be finite and in (0, 1]"; return false; }
    if (!std::isfinite(c.min_p) || !(0.0f <= c.min_p && c.min_p <= 1.0f)) { *why = "min_p must be finite and in [0, 1]"; return false; }
    return true;
}
}  // namespace

extern "C" {

dfl_status dfl_sampler_create(const dfl_sampling_config* cfg, dfl_sampler** out) {
    if (!cfg || !out) return fail(DFL_ERR_BAD_ARG, "sampler_create: null argument");
    *out = nullptr;
    std::string why;
    if (!valid_config(*cfg, &why)) return fail(DFL_ERR_SAMPLING, why);
    auto* s = new dfl_sampler();
    s->cfg = *cfg;
    s->rng.seed(cfg->seed);
    *out = s;
    return DFL_OK;
}
dfl_status dfl_sampler_create_at_draw(const dfl_sampling_config* cfg, uint64_t draws, dfl_sampler** out) {
    dfl_status st = dfl_sampler_create(cfg, out);
    if (st != DFL_OK) return st;
    for (uint64_t i = 0; i < draws; ++i) (*out)->rng.next_u64();
    (*out)->draws = draws;
    return DFL_OK;
}
void dfl_sampler_destroy(dfl_sampler* s) { delete s; }

dfl_status dfl_sampler_set_worker_threads(dfl_sampler* s, uint32_t n) {
    if (!s) return DFL_ERR_BAD_ARG;
    s->workers = n;
    return DFL_OK;
}

uint64_t dfl_sampler_preordered_rows(const dfl_sampler* s) { return s ? s->ord_used.load(std::memory_order_relaxed) : 0; }

dfl_status dfl_sampler_set_row_order(dfl_sampler* s, const float* logits_base, const uint32_t* order_base, uint32_t n_rows,
                                     uint64_t vocab) {
    if (!s) return DFL_ERR_BAD_ARG;
    if (!logits_base || !order_base || n_rows == 0 || vocab == 0) {
        s->ord_logits = nullptr;
        s->ord_base = nullptr;
        s->ord_rows = 0;
        s->ord_vocab = 0;
        return DFL_OK;
    }
    s->ord_logits = logits_base;
    s->ord_base = order_base;
    s->ord_rows = n_rows;
    s->ord_vocab = vocab;
    return DFL_OK;
}
void dfl_sampler_get_config(const dfl_sampler* s, dfl_sampling_config* out) { if (s && out) *out = s->cfg; }
uint64_t dfl_sampler_draws(const dfl_sampler* s) { return s ? s->draws : 0; }
void dfl_sampler_rng_state(const dfl_sampler* s, uint64_t out_state[4]) {
    if (s) std::memcpy(out_state, s->rng.st, 32);
}
uint64_t dfl_splitmix64_next(uint64_t* state) {
    SplitMix64 sm{*state};
    const uint64_t v = sm.next();
    *state = sm.s;
    return v;
}
uint64_t dfl_sampler_next_u64(dfl_sampler* s) { return s->rng.next_u64(); }
double dfl_sampler_next_unit_f64(dfl_sampler* s) { return s->rng.next_unit(); }

dfl_status dfl_sampler_sample(dfl_sampler* s, const float* logits, uint64_t vocab, int32_t* token_out, uint64_t* candidate_index_out) {
    if (!s || !token_out) return fail(DFL_ERR_BAD_ARG, "sampler_sample: null argument");
    if (vocab && !logits) return fail(DFL_ERR_BAD_ARG, "sampler_sample: logits is null");
    uint64_t nan_token = 0, idx = 0;
    SErr e = s->sample(logits, vocab, token_out, &idx, &nan_token);
    if (candidate_index_out) *candidate_index_out = idx;
    return e == S_OK ? DFL_OK : sampling_fail(e, nan_token, -1);
}

dfl_status dfl_sampler_sample_with_distribution(dfl_sampler* s, const float* logits, uint64_t vocab, int32_t* token_out,
                                                uint64_t* candidate_index_out, int32_t* dist_tokens, double* dist_weights, uint64_t cap,
                                                uint64_t* count, double* total_weight) {
    if (!s || !token_out || (vocab && !logits)) return fail(DFL_ERR_BAD_ARG, "sample_with_distribution: null argument");
    uint64_t nan_token = 0;
    Dist d;
    SErr e;
    if (s->cfg.temperature == 0.0f) {
        e = s->diagnose0(logits, vocab, d, &nan_token);
    } else {
        e = s->distribution(logits, vocab, d, &nan_token);
        if (e == S_OK) {
            ++s->draws;
            dfl_sampler::pick(d, s->rng.next_unit());
        }
    }
    if (e != S_OK) return sampling_fail(e, nan_token, -1);
    *token_out = d.sampled;
    if (candidate_index_out) *candidate_index_out = d.index;
    if (count) *count = d.tokens.size();
    if (total_weight) *total_weight = d.total;
    for (uint64_t i = 0; i < d.tokens.size() && i < cap; ++i) {
        if (dist_tokens) dist_tokens[i] = d.tokens[i];
        if (dist_weights) dist_weights[i] = d.weights[i];
    }
    return DFL_OK;
}

dfl_status dfl_greedy_token(const float* logits, uint64_t vocab, int32_t* token_out) {
    if (!token_out || (vocab && !logits)) return fail(DFL_ERR_BAD_ARG, "greedy_token: null argument");
    uint64_t nan_token = 0;
    SErr e = dfl_sampler::greedy(logits, vocab, token_out, &nan_token);
    return e == S_OK ? DFL_OK : sampling_fail(e, nan_token, -1);
}

dfl_status dfl_sampler_couple_sparse(dfl_sampler* s, const float* logits, uint64_t vocab, int32_t proposal_token, const int32_t* cand_tokens,
                                     const double* cand_weights, uint32_t n_cand, int32_t* accepted, int32_t* correction) {
    if (!s || !logits || !accepted || !correction || (n_cand && (!cand_tokens || !cand_weights)))
        return fail(DFL_ERR_BAD_ARG, "couple_sparse: null argument");
    bool acc = false;
    uint64_t nan_token = 0;
    const Xoshiro saved_rng = s->rng;  // an error consumes no RNG state
    const uint64_t saved_draws = s->draws;
    SErr e = s->couple_sparse(logits, vocab, proposal_token, cand_tokens, cand_weights, n_cand, &acc, correction, &nan_token);
    if (e != S_OK) {
        s->rng = saved_rng;
        s->draws = saved_draws;
        return sampling_fail(e, nan_token, -1);
    }
    *accepted = acc ? 1 : 0;
    return DFL_OK;
}

dfl_status dfl_accept_prefix(const int32_t* verified_tokens, uint32_t n_tokens, const float* target_logits, uint64_t n_logits, uint64_t vocab,
                             const dfl_sparse_proposals* proposals, dfl_sampler* sampler, uint64_t remaining_output_budget,
                             const int32_t* stop_ids, uint32_t n_stop_ids, dfl_accept_decision* out) {
    if (!out || !sampler) return fail(DFL_ERR_BAD_ARG, "accept_prefix: null argument");
    std::memset(out, 0, sizeof(*out));
    out->error_row = -1;
    if (n_tokens == 0 || !verified_tokens) return fail(DFL_ERR_BAD_ARG, "invalid DFlash accept-prefix input: missing carry token");
    if (n_tokens > DFL_MAX_BLOCK) return fail(DFL_ERR_BAD_SHAPE, "invalid DFlash accept-prefix input: more than 16 verified tokens");
    if (vocab == 0 || vocab > 0x7fffffffull) return fail(DFL_ERR_BAD_ARG, "invalid DFlash accept-prefix input: invalid vocabulary size");
    if ((uint64_t)n_tokens * vocab != n_logits || !target_logits)
        return fail(DFL_ERR_BAD_SHAPE, "invalid DFlash accept-prefix input: target logits extent mismatch");
    for (uint32_t i = 0; i < n_tokens; ++i)
        if (verified_tokens[i] < 0 || (uint64_t)verified_tokens[i] >= vocab)
            return fail(DFL_ERR_BAD_TOKEN, "verified input token at index " + std::to_string(i) + " is outside the vocabulary");
    const uint32_t n_drafts = n_tokens - 1;
    if (proposals) {
        if (proposals->n_rows != n_drafts) return fail(DFL_ERR_BAD_SHAPE, "invalid DFlash accept-prefix input: proposal row count mismatch");
        for (uint32_t row = 0; row < n_drafts; ++row) {
            if (proposals->tokens[row] != verified_tokens[row + 1])
                return fail(DFL_ERR_BAD_ARG, "proposal row " + std::to_string(row) + " sampled a token that is not the verified draft");
            for (uint32_t c = proposals->cand_offsets[row]; c < proposals->cand_offsets[row + 1]; ++c)
                if (proposals->cand_tokens[c] < 0 || (uint64_t)proposals->cand_tokens[c] >= vocab) {
                    out->error_row = (int32_t)row;
                    return sampling_fail(S_PROPOSAL_RANGE, 0, (int)row);
                }
        }
    }
    auto is_stop = [&](int32_t t) {
        for (uint32_t i = 0; i < n_stop_ids; ++i)
            if (stop_ids[i] == t) return true;
        return false;
    };
    if (is_stop(verified_tokens[0])) { out->stop_reason = DFL_STOP_EOS; return DFL_OK; }
    if (remaining_output_budget == 0) { out->stop_reason = DFL_STOP_TOKEN_LIMIT; return DFL_OK; }

    // The request sampler advances in place and is rolled back on any error (accept.rs:147,176).
    dfl_sampler& next = *sampler;
    next.prepare_rows(target_logits, n_tokens, vocab);
    struct Unprepare {
        dfl_sampler& s;
        ~Unprepare() { s.end_block(); }
    } unprepare{next};
    const Xoshiro saved_rng = sampler->rng;
    const uint64_t saved_draws = sampler->draws;
    auto rollback = [&]() { sampler->rng = saved_rng; sampler->draws = saved_draws; };
    uint32_t n_acc = 0;
    int32_t carry_kind = DFL_CARRY_NONE, carry = 0, stop = DFL_STOP_NONE;
    for (;;) {
        const uint32_t row = n_acc;
        const float* logits = target_logits + (uint64_t)row * vocab;
        uint64_t nan_token = 0, idx = 0;
        if (row == n_drafts) {
            int32_t bonus = 0;
            SErr e = next.sample(logits, vocab, &bonus, &idx, &nan_token);
            if (e != S_OK) { rollback(); out->error_row = (int32_t)row; return sampling_fail(e, nan_token, (int)row); }
            carry_kind = DFL_CARRY_BONUS;
            carry = bonus;
            break;
        }
        const int32_t draft = verified_tokens[row + 1];
        bool accepted = false;
        int32_t correction = 0;
        SErr e;
        if (proposals) {
            const uint32_t c0 = proposals->cand_offsets[row], c1 = proposals->cand_offsets[row + 1];
            e = next.couple_sparse(logits, vocab, proposals->tokens[row], proposals->cand_tokens + c0, proposals->cand_weights + c0, c1 - c0,
                                   &accepted, &correction, &nan_token);
        } else {
            int32_t target = 0;
            e = next.sample(logits, vocab, &target, &idx, &nan_token);
            accepted = target == draft;
            correction = target;
        }
        if (e != S_OK) { rollback(); out->error_row = (int32_t)row; return sampling_fail(e, nan_token, (int)row); }
        if (!accepted) { carry_kind = DFL_CARRY_CORRECTION; carry = correction; break; }
        out->accepted_drafts[n_acc++] = draft;
        if (is_stop(draft)) { stop = DFL_STOP_EOS; break; }
        if (n_acc == remaining_output_budget) { stop = DFL_STOP_TOKEN_LIMIT; break; }
    }
    out->n_accepted = n_acc;
    out->next_carry_kind = carry_kind;
    out->next_carry = carry;
    out->stop_reason = stop;
    out->retain_input_count = 1 + n_acc - (stop != DFL_STOP_NONE ? 1 : 0);
    return DFL_OK;
}

}  // extern "C"
