// Host-side objects behind the opaque C handles: resident target model, per-sequence session,
// verify scratch, drafter and drafter session.  They mirror the reference's MetalModel /
// MetalSession / MetalDFlashVerifyScratch / MetalDFlashHead / MetalDFlashSession
// (crates/qwen-llm/src/metal_forward/mod.rs:443,2095; crates/qwen-llm/src/metal_dflash.rs:4944,5492,6003).
#pragma once
#include <atomic>
#include <functional>
#include <map>
#include <string>
#include <vector>

#include "ops.cuh"

namespace dfl {

dfl_status use_device(int device);
dfl_status check_dev_err(cudaStream_t st, int* dev_err);
dfl_status qmatrix_create(int device, int dtype, uint64_t n_in, uint64_t n_out, const void* data, uint64_t n_bytes, bool on_device,
                          cudaStream_t st, QMatrix* m, bool allow_ts = false, int kb_group = 0);
void qmatrix_release(QMatrix* m);

// Several matrices that consume the same activations and write side by side into one
// partial buffer [splits][16][total_cols].
struct MatGroup {
    std::vector<QMatrix> mats;
    std::vector<uint32_t> col_off;
    uint32_t total_cols = 0;
    uint64_t n_in = 0;
    int splits = 1;
    uint64_t ggml_bytes() const { uint64_t b = 0; for (auto& m : mats) b += m.ggml_bytes(); return b; }
    uint64_t bytes() const { uint64_t b = 0; for (auto& m : mats) b += m.bytes(); return b; }   // as resident in HBM
    void release() { for (auto& m : mats) qmatrix_release(&m); mats.clear(); }
};
dfl_status launch_group(cudaStream_t st, const MatGroup& g, const uint8_t* acts, float* part, const GemmEpilogue& ep, int* err);

struct TensorMap {
    std::map<std::string, const dfl_tensor*> t;
    const dfl_tensor* find(const std::string& n) const { auto it = t.find(n); return it == t.end() ? nullptr : it->second; }
};
// Builds a MatGroup from named tensors [n_in, n_out]; consecutive tensors of one dtype are
// concatenated row-wise into one resident matrix (one kernel launch instead of several).
dfl_status build_group(int device, cudaStream_t st, const TensorMap& tm, const std::vector<std::string>& names, uint64_t n_in,
                       const std::vector<uint64_t>& n_outs, MatGroup* out, bool allow_ts = false, int kb_group = 0);
// Uploads a small tensor as f32 (norm weights, biases, f32 projections); any ggml dtype.
dfl_status upload_f32(int device, cudaStream_t st, const TensorMap& tm, const std::string& name, uint64_t n_expected, float** out);

struct LayerW {
    bool is_attn = false;
    float *attn_norm_w = nullptr, *post_norm_w = nullptr;
    // full attention
    MatGroup qkv;  // q (interleaved q|gate per head), k, v
    MatGroup wo;
    float *q_norm_w = nullptr, *k_norm_w = nullptr;
    // gated delta net
    MatGroup in_qkv_z;  // attn_qkv then attn_gate
    MatGroup w_out;
    float *w_ab = nullptr;  // [2 n_v][H]: ssm_alpha rows, then ssm_beta rows
    float *a_log = nullptr, *dt_bias = nullptr, *conv_w = nullptr, *ssm_norm_w = nullptr;
    // dense FFN
    MatGroup gate_up;
    MatGroup down;
    // routed experts + shared expert (arch.expert_count > 0): gate|up of all experts and of the shared expert in
    // one group (columns: E*F' expert gates, F_sh shared gate, E*F' expert ups, F_sh shared up), the experts' down
    // projections as one matrix over n_in = E*F', the shared expert's down, and the f32 router with the shared
    // expert's gate vector as its last row [E + 1][H]
    MatGroup moe_gate_up, moe_down, moe_down_sh;
    float* router_w = nullptr;
};

}  // namespace dfl

struct dfl_session;

namespace dfl {
// expert parallelism (ep_nccl.cpp)
dfl_status ep_unique_id(uint8_t* id_out);
dfl_status ep_comm_create(int rank, int world, const uint8_t* id_bytes, void** comm_out);
void ep_comm_destroy(void* comm, bool aborted);
dfl_status ep_all_reduce_sum(void* comm, float* buf, size_t count, cudaStream_t st);
// peer-memory combine (ep_combine.cu): every rank's exchange buffer - receive slots [2 parities][world][16][H] f32,
// then flags [2][world][ctas] u32 at flags_off - mapped into this process
constexpr int EP_MAX_WORLD = 8;
struct EpPeers {
    float* base[EP_MAX_WORLD];
    uint64_t flags_off;
};
inline int ep_combine_ctas(uint64_t n_out) { return (int)((MAX_ROWS * n_out / 4 + 255) / 256); }
inline uint64_t ep_recv_floats(int world, uint64_t n_out) { return 2ull * (uint64_t)world * MAX_ROWS * n_out; }
dfl_status ep_p2p_exchange(void* comm, int rank, int world, void* local, cudaStream_t st, void** peers_out);
void ep_p2p_close(int rank, int world, void* const* peers);
bool ep_barrier_bounded(void* comm, cudaStream_t st, uint32_t timeout_ms);
dfl_status launch_ep_push_sum(cudaStream_t st, const float* part, int splits, const int32_t* splits_dev, uint64_t n_out, const EpPeers& peers,
                              int rank, int world, uint32_t seq, const int* abort_host_dev, int* err);
// host watchdog over a pass that contains collectives (ep_nccl.cpp)
struct EpWatchHooks {
    std::function<int()> query;
    std::function<int()> async_error;
    std::function<void()> abort;
};
dfl_status ep_watch_core(const EpWatchHooks& h, uint32_t timeout_ms, uint32_t poll_us, bool* aborted);
dfl_status ep_watch_stream(void* comm, cudaStream_t st, cudaEvent_t ev, volatile int* abort_word, bool* aborted);
dfl_status session_drain(dfl_session* s);
}  // namespace dfl

struct dfl_model {
    int device = 0;
    // expert parallelism: this rank holds experts [ep_e0, ep_e0 + ep_n) of every layer (all of them when ep_world == 1)
    // and, on rank 0 only, the shared expert; each block's output is summed over the ranks
    int ep_rank = 0, ep_world = 1;
    uint32_t ep_e0 = 0, ep_n = 0, ep_fs = 0;
    void* ep_comm = nullptr;
    mutable std::atomic<bool> ep_dead{false};   // the watchdog aborted the communicator: every later pass is refused
    // peer-memory combine: the exchange buffers of all ranks (own one at [ep_rank]), the combine counter every rank
    // advances alike, and the host-mapped word the watchdog raises to end waiting kernels
    bool ep_p2p = false;
    dfl::EpPeers ep_peers{};
    mutable uint32_t ep_seq = 0;
    int* ep_abort_host = nullptr;
    int* ep_abort_dev = nullptr;
    int act_layout = dfl::ACT_F16;  // packed-activation format all its GEMMs consume (follows the kernel family)
    dfl_arch arch{};
    std::vector<dfl::LayerW> layers;
    uint8_t* embd_ggml = nullptr;  // token_embd in ggml layout (row gather)
    int embd_dtype = 0;
    dfl::MatGroup lm_head;
    float* out_norm_w = nullptr;
    uint64_t verify_weight_bytes = 0;     // ggml bytes one verify pass touches
    uint64_t verify_resident_bytes = 0;   // the same matrices as they are resident (Q6_K tiles hold a byte per code)
    std::vector<void*> allocs;
    int n_gdn = 0, n_attn = 0;
    dfl::AttnGeom attn_geom() const {
        dfl::AttnGeom g;
        g.n_q = (int)arch.n_q_heads; g.n_kv = (int)arch.n_kv_heads; g.hd = (int)arch.attn_head_dim;
        g.n_rot = (int)((float)arch.attn_head_dim * arch.partial_rotary_factor);
        g.theta = arch.rope_theta; g.eps = 1e-6f;
        return g;
    }
    dfl::GdnGeom gdn_geom() const {
        dfl::GdnGeom g;
        g.n_v = (int)arch.gdn_n_v_heads; g.n_k = (int)arch.gdn_n_k_heads; g.hd = (int)arch.gdn_head_dim; g.conv_k = (int)arch.gdn_conv_kernel;
        return g;
    }
};

struct dfl_session {
    const dfl_model* m = nullptr;
    uint32_t kv_capacity = 0;
    bool kv_f16 = false;
    int kv_mode = dfl::KV_F32_ROWS;   // storage of the K / V caches (ops.cuh KvMode); tiled only for f16, 128-wide heads, groups of four
    uint32_t kv_n_pos = 0;
    bool poisoned = false;
    bool fail_next = false;
    std::vector<void*> k_cache, v_cache;  // per attention layer: [capacity][n_kv][hd] rows, or tiles of 128 positions per KV head (kv_mode)
    std::vector<float*> conv;             // per GDN layer: [3][conv_dim]
    std::vector<float*> ssm[2];           // per GDN layer, double buffered: [n_v][128][128]
    std::vector<int> ssm_cur;
    float* attn_partials = nullptr;
    cudaStream_t st = nullptr;
    int* err = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    // side stream for the branches of a layer that only depend on the layer's normalised input (the GDN z and
    // alpha / beta projections, the expert router): they run beside the main projection instead of after it
    cudaStream_t st_side = nullptr, st_side2 = nullptr;
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr, ev_join2 = nullptr, ev_watch = nullptr;
};

struct dfl_scratch {
    const dfl_model* m = nullptr;
    uint32_t block_size = 0, k_layers = 0;
    float *x = nullptr, *xn = nullptr, *part = nullptr, *sumsq = nullptr;
    uint8_t *acts_h = nullptr, *acts_f = nullptr, *acts_v = nullptr;
    float *q_rot = nullptr, *gate = nullptr;
    // per GDN layer, kept for rollback
    std::vector<float*> qkv_raw, conv_pre, q_n, k_n, v, ab;
    float *logits = nullptr, *gap = nullptr;
    int32_t* argmax = nullptr;
    // routed experts: router logits [16][E + 1], dense route weights [16][E], shared-expert gates [16], chosen ids [16][k]
    float *route_logits = nullptr, *route_w = nullptr, *route_sg = nullptr, *moe_out = nullptr;
    int32_t* route_idx = nullptr;
    int32_t *moe_tile_map = nullptr, *moe_n_tiles = nullptr, *moe_kb_map = nullptr;   // row tiles of the gate|up matrix the block's routing needs
    void* am_scratch = nullptr;
    float* capture = nullptr;  // [16][k][H]
    int32_t* tokens_dev = nullptr;
    int32_t* pinned_i = nullptr;  // [16] tokens in, [16] argmax out
    float* pinned_f = nullptr;    // [16] gaps
    float* pinned_logits = nullptr;  // [block][vocab], made on first use by the sampled outer loop
    // rows ordered on the device for the host sampler (sortrows.cu): destination on the host (null = off), device
    // order [block][vocab] and the sort's scratch (made on first use), and a pinned destination of the outer loop
    uint32_t* order_host = nullptr;
    uint32_t* order_dev = nullptr;
    void* sort_scratch = nullptr;
    uint32_t* pinned_order = nullptr;
    uint32_t last_n = 0, last_start = 0;
    uint32_t last_n_verify = 0;   // rows of the last verify (last_n shrinks to n_keep after a partial restore)
    bool have_block = false;
    uint64_t part_floats = 0;
    std::vector<void*> allocs;
};

namespace dfl {
// One packed forward of n <= 16 tokens at positions start..start+n-1 (the body shared by
// dfl_packed_verify, dfl_single_token and dfl_prefill).  Leaves argmax/gap/logits/capture on the device.
dfl_status verify_core(const dfl_model* m, dfl_session* s, dfl_scratch* sc, const uint32_t* layer_ids, uint32_t n_ids,
                       const int32_t* tokens, uint32_t n, uint32_t start, bool want_head);
dfl_status session_guard(const dfl_model* m, dfl_session* s, const char* what);
// the drafter session's part of a session snapshot (drafter.cu)
uint64_t dsession_snapshot_bytes(const dfl_dsession* ds);
dfl_status dsession_snapshot_write(dfl_dsession* ds, uint8_t* dst, uint32_t* cols_out);
dfl_status dsession_snapshot_read(dfl_dsession* ds, const uint8_t* src, uint32_t cols, uint64_t n_bytes);
dfl_status dsession_snapshot_validate(const dfl_dsession* ds, uint32_t cols, uint64_t n_bytes);
void dsession_identity(const dfl_dsession* ds, uint32_t out[3]);
const dfl_model* dsession_target(const dfl_dsession* ds);
}  // namespace dfl
