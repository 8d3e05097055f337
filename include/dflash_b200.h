/*
 * dflash_b200 — C ABI of the B200 (sm_100a) DFlash speculative-decoding step.
 *
 * Every entry point replaces one call the reference engine (brittlewis12/qwen-llm)
 * makes from Rust into its Metal backend; the reference item is cited beside each
 * declaration as `crate-relative path:line`.  Conventions, mirroring
 * crates/qwen-llm/src/metal_dflash.rs:2698-2732 (DFlashError) and
 * crates/qwen-llm/src/metal/completion.rs:18 (checked waits):
 *
 *   - every function returns a dfl_status (0 == success); nothing throws across
 *     the boundary; dfl_last_error() gives the text of the calling thread's last
 *     failure;
 *   - handles are opaque; weights are immutable and shareable, a session /
 *     drafter session / scratch is exclusively owned by the caller for the
 *     duration of a call (one caller thread per session);
 *   - calls are synchronous: they return after the device work completed and its
 *     status was checked, so host outputs are valid on return;
 *   - a failed route status or device error poisons the session
 *     (crates/qwen-llm/src/metal_forward/mod.rs:2161-2170): later calls fail with
 *     DFL_ERR_POISONED;
 *   - there is no CPU fallback: without a CUDA device compute calls fail with
 *     DFL_ERR_NO_DEVICE.
 */
#ifndef DFLASH_B200_H
#define DFLASH_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum dfl_status {
    DFL_OK = 0,
    DFL_ERR_BAD_ARG = 1,       /* null pointer, out-of-range scalar */
    DFL_ERR_BAD_SHAPE = 2,     /* DFlashError::BadShape{kernel,detail} */
    DFL_ERR_UNSUPPORTED = 3,   /* dtype / geometry the kernels do not cover */
    DFL_ERR_CUDA = 4,          /* a CUDA runtime call or a kernel failed */
    DFL_ERR_NO_DEVICE = 5,     /* no usable CUDA device: compute refused */
    DFL_ERR_OOM = 6,
    DFL_ERR_POISONED = 7,      /* session poisoned by an earlier failure */
    DFL_ERR_CTX_OVERFLOW = 8,  /* DFlashError::CtxOverflow, metal_dflash.rs:5666 */
    DFL_ERR_KV_STATE = 9,      /* kv_n_pos / capacity guard wall, metal_dflash.rs:9079-9186 */
    DFL_ERR_BAD_TOKEN = 10,    /* ForwardError::BadToken, forward.rs:24 */
    DFL_ERR_SAMPLING = 11,     /* SamplingError / DFlashAcceptError */
    DFL_ERR_TIMEOUT = 12,      /* a bounded device-side wait gave up */
    DFL_ERR_MISSING_TENSOR = 13,
    DFL_ERR_ROUTE_STATUS = 14, /* expert routing reported NONFINITE (kernels/moe.metal:355-360); poisons the session */
    DFL_ERR_COLLECTIVE = 15    /* expert-parallel watchdog: a collective failed or did not complete; communicator aborted */
} dfl_status;

/* ggml type ids (crates/qwen-llm/src/tensor.rs:159 `storage_layout`). */
typedef enum dfl_dtype {
    DFL_F32 = 0,
    DFL_F16 = 1,
    DFL_Q8_0 = 8,   /* 34 B / 32 weights  */
    DFL_Q4_K = 12,  /* 144 B / 256 weights */
    DFL_Q5_K = 13,  /* 176 B / 256 weights */
    DFL_Q6_K = 14,  /* 210 B / 256 weights */
    DFL_BF16 = 30
} dfl_dtype;

/* One named tensor in ggml storage order (ne[0] fastest).  Mirrors TensorDesc,
 * crates/qwen-llm/src/tensor.rs.  `data` is a host pointer unless
 * `on_device` != 0, in which case it is a device pointer on the model's GPU. */
typedef struct dfl_tensor {
    const char* name;
    int32_t dtype;       /* dfl_dtype */
    int32_t n_dims;      /* 1..3 */
    uint64_t shape[4];   /* ne[0..n_dims) */
    const void* data;
    uint64_t n_bytes;
    int32_t on_device;
    int32_t _pad;
} dfl_tensor;

/* Architecture of the hybrid target.  Mirrors `Arch`,
 * crates/qwen-llm/src/model.rs:40-70. */
typedef struct dfl_arch {
    uint32_t n_layer;
    uint32_t hidden_size;
    uint32_t intermediate_size;
    uint32_t vocab_size;
    uint32_t full_attention_interval;
    uint32_t n_q_heads;
    uint32_t n_kv_heads;
    uint32_t attn_head_dim;
    float rope_theta;
    float partial_rotary_factor;
    uint32_t gdn_n_v_heads;
    uint32_t gdn_n_k_heads;
    uint32_t gdn_head_dim;
    uint32_t gdn_conv_kernel;
    uint32_t expert_count;                       /* 0 on dense models */
    uint32_t expert_used_count;
    uint32_t expert_feed_forward_length;
    uint32_t expert_shared_feed_forward_length;
} dfl_arch;

#define DFL_MAX_TARGET_LAYERS 8
#define DFL_MAX_BLOCK 16
#define DFL_MAX_DRAFTER_LAYERS 16

/* Drafter description.  Mirrors `DFlashConfig` + `DFlashHead.target_layer_ids` +
 * per-layer `is_swa`, crates/qwen-llm/src/loader.rs:340-409. */
typedef struct dfl_dflash_config {
    uint32_t n_layer;
    uint32_t hidden_size;
    uint32_t intermediate_size;
    uint32_t n_q_heads;
    uint32_t n_kv_heads;
    uint32_t head_dim;
    float rope_theta;
    float rms_norm_eps;
    uint32_t causal;
    uint32_t swa_window;
    uint32_t block_size;
    int32_t mask_token_id;
    uint32_t n_target_layers;                          /* K */
    uint32_t target_layer_ids[DFL_MAX_TARGET_LAYERS];
    uint32_t layer_is_swa[DFL_MAX_DRAFTER_LAYERS];
    /* DFlash 2 path selector (loader.rs:371-376, metadata dflash.selector_rank / dflash.selector_top_k); both 0 on
     * a DFlash 1 drafter.  With a selector the tensor table must hold selector_hidden.weight [H, rank],
     * selector_predecessor.weight and selector_successor.weight [rank, vocab] (loader.rs:1182-1230). */
    uint32_t selector_rank;
    uint32_t selector_top_k;   /* only 16 is supported, as in the reference (metal_dflash.rs:5011-5017) */
} dfl_dflash_config;

typedef struct dfl_model dfl_model;       /* MetalModel          metal_forward/mod.rs:443  */
typedef struct dfl_session dfl_session;   /* MetalSession        metal_forward/mod.rs:2095 */
typedef struct dfl_drafter dfl_drafter;   /* MetalDFlashHead     metal_dflash.rs:4944      */
typedef struct dfl_dsession dfl_dsession; /* MetalDFlashSession  metal_dflash.rs:5492      */
typedef struct dfl_scratch dfl_scratch;   /* MetalDFlashVerifyScratch + LayerMajorScratch
                                             metal_dflash.rs:6003, :8025                   */
typedef struct dfl_qmatrix dfl_qmatrix;   /* one resident quantised matrix (MetalTensor)   */
typedef struct dfl_sampler dfl_sampler;   /* Sampler             sampling.rs:305           */
typedef struct dfl_codebook dfl_codebook; /* DFlash2Codebook     metal_dflash.rs:3163      */
typedef struct dfl_gguf dfl_gguf;         /* GgufFile            gguf.rs:154               */

/* ---- library / diagnostics --------------------------------------------- */
const char* dfl_version(void);
const char* dfl_last_error(void);
/* Number of usable CUDA devices (0 when the driver or a device is missing). */
int32_t dfl_device_count(void);
/* How this process's host threads wait for the device in every synchronising call of this library: 0 the driver's
 * default (spins while contexts are fewer than cores), 1 spin, 2 yield, 3 block on an OS primitive.  Blocking frees the
 * core for the sampler's worker threads when many driving threads share a host (one per sequence, several ranks); it
 * costs a wake-up per wait, so a single driving thread is faster with the default.  The environment variable
 * DFL_HOST_WAIT=auto|spin|yield|block sets the initial policy.  Takes effect at each device's next use. */
dfl_status dfl_set_host_wait(int32_t mode);
/* Kernel launches this library issued on the calling process since load. */
uint64_t dfl_launch_count(void);
/* Per-kernel device timing of the few-row GEMM (the reference reads per-phase GPU time from
 * GPUStartTime/GPUEndTime, metal_dflash.rs:5608-5634).  Between begin and end every GEMM launch is
 * bracketed by CUDA events on its own stream; end synchronises them and returns the summed kernel
 * time, the launch count and the ggml weight bytes those launches streamed. */
void dfl_gemm_timing_begin(void);
dfl_status dfl_gemm_timing_end(double* ms_total, uint64_t* n_launches, uint64_t* weight_bytes);

/* ---- few-row quantised GEMM (the weight-streaming hot kernel) ----------
 * Replaces encode_mat_mat_dispatch / kernel_mat_mat_*_fewrow_gen,
 * crates/qwen-llm/src/metal_forward/dispatch.rs:345-433,
 * kernels/mat_mat_fewrow_gen.metal:374-474.
 * W is row-major [n_out][n_in] in ggml blocks; y[r, o] = sum_i x[r, i] W[o, i]. */
dfl_status dfl_qmatrix_create(int32_t device, int32_t dtype, uint64_t n_in, uint64_t n_out,
                              const void* data, uint64_t n_bytes, int32_t on_device,
                              dfl_qmatrix** out);
void dfl_qmatrix_destroy(dfl_qmatrix* m);
/* Which kernel serves this matrix: 2 the tcgen05 / tensor-memory few-row GEMM (Q4_K, Q5_K, Q6_K, bf16, and Q8_0 whose
 * block scales are finite and at most 256 in magnitude), 1 the mma.sync few-row GEMM, 0 the f32 small-matrix kernel. */
int32_t dfl_qmatrix_engine(const dfl_qmatrix* m);
/* Decode the resident (re-tiled) matrix back to f32 [n_out][n_in] on the host:
 * proves the integer unpack equals ggml's (codec.rs:287 dequant_to_f32). */
dfl_status dfl_qmatrix_dequant(const dfl_qmatrix* m, float* out_host, uint64_t n_floats);
/* x_host [n_rows][n_in] f32, y_host [n_rows][n_out] f32, 1 <= n_rows <= 16. */
dfl_status dfl_fewrow_matmul(const dfl_qmatrix* m, const float* x_host, int32_t n_rows,
                             float* y_host);
/* Row argmax with lowest-index ties and (top1 - top2) gap; replaces
 * encode_argmax_top2_f32, kernels/elementwise.metal:1231-1286. */
dfl_status dfl_argmax_top2(int32_t device, const float* logits_host, int32_t n_rows,
                           uint64_t vocab, int32_t* argmax_out, float* gap_out);
/* The same row argmax for a caller that must not allocate device memory or
 * wait for the GPU: an ordinary host thread that holds a lock the CUDA
 * allocator may also need, or a serving loop with a fixed memory budget.  (It
 * is not for code inside a stream's host callback: CUDA forbids runtime calls
 * there, and this function makes several.)  This entry point has no counterpart
 * in the reference; it exists for such callers.  logits_dev [n_rows][ld] f32,
 * argmax_dev [n_rows] and gap_dev [n_rows] are the caller's own buffers on
 * `device`; `stream` is a cudaStream_t (NULL = the default stream).  The call
 * makes `device` the calling thread's current device and leaves it so, enqueues
 * two kernels on `stream` and returns without waiting: results are valid once
 * the stream reaches that point.  It calls no allocation or free routine; its
 * per-row partial results live in one fixed 16 KiB array inside the library,
 * sized for n_rows <= 16 (larger n_rows is refused with DFL_ERR_BAD_SHAPE).
 * The first call on each device also looks up the array's address (and may
 * make the driver load the library's kernels, which is not allocation-free from
 * the driver's point of view), so make one call per device before starting a
 * stream capture or entering the section that must not allocate.  Every call on
 * a device shares that array and each call overwrites the part it uses before
 * reading it, so nothing needs clearing; but two calls whose kernels can
 * overlap (different streams, or different threads on different streams)
 * race on it: keep calls on one device in stream order. */
dfl_status dfl_argmax_top2_static(int32_t device, const float* logits_dev, int32_t n_rows,
                                  uint64_t vocab, uint64_t ld, int32_t* argmax_dev,
                                  float* gap_dev, void* stream);

/* ---- the CPU-runnable verify/accept case: two chained few-row GEMMs + greedy acceptance ---
 * logits = head(x W1^T); argmax per row; greedy prefix accept against drafts.
 * Device-resident pipeline object so the timed region has no allocation. */
typedef struct dfl_c1 dfl_c1;
dfl_status dfl_c1_create(const dfl_qmatrix* w1, const dfl_qmatrix* head, dfl_c1** out);
void dfl_c1_destroy(dfl_c1* p);
/* Host-to-host call: copies x in, runs both GEMMs + argmax, copies results out.
 * logits_host may be NULL.  n_accepted = longest j with draft[j]==argmax[j]. */
dfl_status dfl_c1_step(dfl_c1* p, const float* x_host, int32_t n_rows, const int32_t* draft_ids,
                       int32_t* argmax_out, float* gap_out, int32_t* n_accepted,
                       float* logits_host);
/* Same work with x already resident (uploaded by dfl_c1_upload); returns the
 * device time of the kernels alone in milliseconds (CUDA events). */
dfl_status dfl_c1_upload(dfl_c1* p, const float* x_host, int32_t n_rows);
dfl_status dfl_c1_run_resident(dfl_c1* p, int32_t n_rows, int32_t iters, float* ms_total);

/* ---- model / drafter / sessions ---------------------------------------- */
/* MetalModel::load  metal_forward/mod.rs:443-454 (tensor names follow
 * crates/qwen-llm/src/loader.rs:438-611).  With arch.expert_count > 0 every
 * layer's FFN is the routed-expert block of forward.rs:749-824 and the table
 * must hold ffn_gate_inp, ffn_{gate,up,down}_exps (experts stacked along the
 * last ggml dimension), ffn_gate_inp_shexp and ffn_{gate,up,down}_shexp;
 * expert widths must be multiples of 256 and the matrices Q4_K / Q5_K / Q6_K. */
dfl_status dfl_model_create(int32_t device, const dfl_arch* arch, const dfl_tensor* tensors,
                            uint64_t n_tensors, dfl_model** out);
void dfl_model_destroy(dfl_model* m);
/* Bytes of quantised weights one verify step streams (the roofline numerator). */
uint64_t dfl_model_verify_weight_bytes(const dfl_model* m);
/* The same matrices counted as they are resident in HBM: equal to the above except that Q6_K tiles of the
 * tensor-memory GEMM hold one six-bit code per byte (274 bytes per 256 weights against ggml's 210). */
uint64_t dfl_model_verify_resident_bytes(const dfl_model* m);
/* Expert parallelism for routed-expert models (one process per GPU of one node).
 * Rank r of ep_world keeps experts [r*E/ep_world, (r+1)*E/ep_world) of every layer
 * (rank 0 also the shared expert), everything else is replicated.  Each
 * routed-expert block ends with a combine over peer memory: every rank sums its
 * own slices and stores its [16][hidden] result into every rank's receive buffer
 * (plain peer stores over NVLink, per-CTA sequence flags), and the layer's glue
 * kernel adds the ranks' slots in rank order, so every rank returns the same
 * bits.  `tensors` is the full table on every rank.  The 128-byte id comes from
 * dfl_ep_unique_id on one rank and is distributed by the caller; all ranks must
 * call dfl_model_create_ep together and then issue the same verify calls in the
 * same order, one pass at a time per model.  NCCL (loaded at run time,
 * libnccl.so.2) carries the bootstrap - the exchange of the buffers' inter-process
 * handles - and, with DFL_EP_COMBINE=nccl in the environment, the sum itself as
 * an all-reduce (kept for comparison).  At most 8 ranks. */
dfl_status dfl_ep_unique_id(uint8_t* id_out_128);
dfl_status dfl_model_create_ep(int32_t device, const dfl_arch* arch, const dfl_tensor* tensors,
                               uint64_t n_tensors, int32_t ep_rank, int32_t ep_world,
                               const uint8_t* nccl_id_128, dfl_model** out);
/* Host watchdog of expert-parallel passes.  Every call that waits for a pass of an
 * expert-parallel model polls an event instead of blocking, asks the communicator
 * for an asynchronous error between polls, and gives up after DFL_EP_TIMEOUT_MS
 * (environment, default 30000): the communicator is aborted, the call returns
 * DFL_ERR_COLLECTIVE, the session is poisoned and every later pass on the model
 * is refused with the same status.  dfl_ep_watchdog_selftest drives the same
 * polling loop with scripted actions and no GPU: scenario 0 = the pass completes
 * after `after_polls` polls (expects DFL_OK, no abort), 1 = the communicator
 * reports an asynchronous error at poll `after_polls`, 2 = the pass never
 * completes (runs into timeout_ms), 3 = the pass itself fails with a CUDA error.
 * *aborted_out = how often the abort action ran (0 or 1). */
dfl_status dfl_ep_watchdog_selftest(int32_t scenario, uint32_t after_polls, uint32_t timeout_ms,
                                    int32_t* aborted_out);

/* MetalDFlashHead::load  metal_dflash.rs:4944-5050 (names loader.rs:1179-1230). */
dfl_status dfl_drafter_create(const dfl_model* target, const dfl_dflash_config* cfg,
                              const dfl_tensor* tensors, uint64_t n_tensors, dfl_drafter** out);
void dfl_drafter_destroy(dfl_drafter* d);
uint64_t dfl_drafter_weight_bytes(const dfl_drafter* d);

/* MetalSession::fresh(ctx, model, kv_capacity)  metal_forward/mod.rs:2238-2391.
 * kv_f16 != 0 stores K/V as fp16 (the reference GPU layout, mod.rs:2330-2341);
 * 0 stores f32 (the CPU oracle's layout, forward.rs:1142-1151).  An fp16 cache of
 * 128-wide heads in GQA groups of four is stored as position-major rows below
 * 16384 positions of capacity and as 128-position tiles in the tensor cores'
 * operand layout from there on (the long-context attention kernel); the choice is
 * fixed per session, invisible through this interface (dfl_session_read_kv and
 * snapshots speak position-major rows for both) and can be forced with
 * DFL_ATTN_TILED=1 / 0 in the environment. */
dfl_status dfl_session_create(const dfl_model* m, uint32_t kv_capacity, int32_t kv_f16,
                              dfl_session** out);
void dfl_session_destroy(dfl_session* s);
uint32_t dfl_session_kv_n_pos(const dfl_session* s);
int32_t dfl_session_poisoned(const dfl_session* s);
/* Test hook mirroring completion::fail_next_completion_check
 * (metal/completion.rs:41-66): the next completion check on this session
 * reports failure without touching the GPU. */
void dfl_session_fail_next_completion(dfl_session* s);
/* Read back recurrent state for bitwise comparisons (tests.rs:7049-7094). */
dfl_status dfl_session_read_gdn_state(const dfl_session* s, uint32_t gdn_index, float* ssm_out,
                                      uint64_t n_ssm, float* conv_out, uint64_t n_conv);
dfl_status dfl_session_read_kv(const dfl_session* s, uint32_t attn_index, uint32_t pos,
                               float* k_out, float* v_out, uint64_t n);

/* ---- session snapshots (SessionSnapshot, metal_forward/session.rs:13-94) ---- */
#define DFL_SNAPSHOT_LAYOUT_VERSION 2
typedef struct dfl_snapshot_identity { /* SnapshotAbi  session.rs:27-37 */
    uint32_t layout_version;
    uint32_t n_attn_layers;
    uint32_t n_gdn_layers;
    uint32_t kv_dim_elements;
    uint32_t kv_bytes_per_token;
    uint32_t kv_storage_kind; /* 0 = f32, 1 = f16 */
    uint32_t gdn_state_elements_per_layer;
    uint32_t gdn_conv_elements_per_layer;
} dfl_snapshot_identity;
dfl_status dfl_session_snapshot_identity(const dfl_model* m, const dfl_session* s,
                                         dfl_snapshot_identity* out);
/* Bytes a snapshot of the session's current prefix takes (with the drafter's context tail when
 * ds != NULL); 0 on a bad argument. */
uint64_t dfl_session_snapshot_bytes(const dfl_model* m, const dfl_session* s, const dfl_dsession* ds);
/* Writes the state after the kv_n_pos tokens consumed so far into `blob`: header with the
 * identity, K and V packed to the prefix, GDN conv and recurrent state, and (ds != NULL) the
 * drafter context a restored request can still see (every column, or the last swa_window
 * columns of an all-sliding-window drafter, metal_dflash.rs:103-140).  Token ids, a pending
 * token and final logits stay with the caller, as in the reference's prefix cache. */
dfl_status dfl_session_snapshot(const dfl_model* m, dfl_session* s, dfl_dsession* ds, void* blob,
                                uint64_t cap, uint64_t* written);
/* Restores into a session of the same model and KV storage (identity checked, section lengths
 * checked, prefix <= kv_capacity).  Continuing from the restored session is bitwise equal to
 * continuing from the session the snapshot was taken from. */
dfl_status dfl_session_restore_snapshot(const dfl_model* m, dfl_session* s, dfl_dsession* ds,
                                        const void* blob, uint64_t n_bytes);

/* When order_host is not NULL, every later dfl_packed_verify on this scratch that returns logits to the host also
 * orders each returned row on the device - token ids by descending logit in the f32 total order, ties by ascending
 * token - and copies the [n][vocab] order to order_host (u32, caller-owned, at least block_size * vocab entries;
 * pinned memory recommended) in the same call.  NULL switches it off.  The first registration on a scratch allocates
 * the device side of the ordering (5 x block_size x vocab x 4 bytes) and can fail with DFL_ERR_OOM; nothing is
 * registered then. */
dfl_status dfl_scratch_set_order_host(dfl_scratch* sc, uint32_t* order_host);
/* The same ordering on rows given by the host (host-to-host test entry): order_out [n_rows][vocab]. */
dfl_status dfl_sort_rows_desc(int32_t device, const float* logits_host, int32_t n_rows, uint64_t vocab,
                              uint32_t* order_out);

/* MetalDFlashVerifyScratch::fresh + MetalDFlashLayerMajorScratch::fresh
 * metal_dflash.rs:6003-6075, :8025. */
dfl_status dfl_scratch_create(const dfl_model* m, uint32_t block_size, uint32_t n_capture_layers,
                              dfl_scratch** out);
void dfl_scratch_destroy(dfl_scratch* s);

/* encode_packed_verify_layer_major_inner  metal_dflash.rs:10696-10719.
 * tokens[n] = [carry, drafts...]; requires kv_n_pos == start_position and
 * start_position + n <= kv_capacity.  Writes argmax_out[n], gap_out[n]
 * (top1 - top2), optional logits_host[n * vocab]; captures hidden rows of
 * `layer_ids` into the scratch as [n][k][H]. */
dfl_status dfl_packed_verify(const dfl_model* m, dfl_session* s, dfl_scratch* sc,
                             const uint32_t* layer_ids, uint32_t n_layer_ids,
                             const int32_t* tokens, uint32_t n, uint32_t start_position,
                             int32_t* argmax_out, float* gap_out, float* logits_host);
/* The same call with the reference's n_eff_override argument spelled out
 * (metal_dflash.rs:9055-9094): n_eff_override < 0 is None (the chain is the
 * scratch's block size), otherwise the effective chain length in [1, block];
 * n_tokens must equal the resolved length. */
dfl_status dfl_packed_verify_n_eff(const dfl_model* m, dfl_session* s, dfl_scratch* sc,
                                   const uint32_t* layer_ids, uint32_t n_layer_ids,
                                   const int32_t* tokens, uint32_t n_tokens, uint32_t start_position,
                                   int32_t n_eff_override, int32_t* argmax_out, float* gap_out,
                                   float* logits_host);
/* Copy captured hidden rows [n][k][H] of the last verify to the host. */
dfl_status dfl_scratch_read_capture(const dfl_scratch* sc, uint32_t n, float* out_host,
                                    uint64_t n_floats);
/* Expert ids the last routed-expert layer of the last verify chose, [n][expert_used_count] in
 * choice order, -1 for a row that was not routed (moe_topk_idx of MetalDFlashLayerMajorScratch,
 * metal_dflash.rs:7240-7443). */
dfl_status dfl_scratch_read_route(const dfl_scratch* sc, uint32_t n, int32_t* idx_out, uint64_t n_idx);
/* Failure-path probe: runs a one-thread kernel on the session's stream that waits, with a limit
 * of `polls` polls (1..65536), on a barrier nobody arrives at.  The wait runs out, the kernel
 * records that in the session's error word and returns normally; the call then reports
 * DFL_ERR_TIMEOUT and the session is poisoned, exactly as when a bounded wait inside a GEMM
 * gives up (the reference's completion check, metal/completion.rs:18, + poisoning,
 * metal_forward/mod.rs:2161-2170). */
dfl_status dfl_session_probe_wait_timeout(const dfl_model* m, dfl_session* s, uint32_t polls);

/* encode_restore_after_partial_accept_inner  metal_dflash.rs:15649-15777:
 * n_keep in [1, n]; GDN state / conv := state after n_keep tokens of the last
 * verify block; kv_n_pos := start_position + n_keep. */
dfl_status dfl_restore_partial(const dfl_model* m, dfl_session* s, dfl_scratch* sc,
                               uint32_t n_keep, uint32_t start_position);
/* ... with n_eff_override as above; it must resolve to the same length as the verify being
 * undone (metal_dflash.rs:15655-15682). */
dfl_status dfl_restore_partial_n_eff(const dfl_model* m, dfl_session* s, dfl_scratch* sc,
                                     uint32_t n_keep, uint32_t start_position, int32_t n_eff_override);
/* encode_restore_to_pre_block  metal_dflash.rs:15789. */
dfl_status dfl_restore_pre_block(const dfl_model* m, dfl_session* s, dfl_scratch* sc,
                                 uint32_t start_position);

/* MetalForward::single_token_with_multi_hidden  metal_forward/token.rs:984.
 * logits_host (optional) [vocab]; hidden_host (optional) [n_layer_ids][H]. */
dfl_status dfl_single_token(const dfl_model* m, dfl_session* s, dfl_scratch* sc,
                            const uint32_t* layer_ids, uint32_t n_layer_ids, int32_t token,
                            uint32_t position, float* logits_host, float* hidden_host);
/* prefill_tokens_with_multi_hidden  metal_dflash.rs:10779-10787: feeds ids in
 * blocks of <=16 through the verify path; hidden_host (optional) [n][k][H] with
 * k = the scratch's capture slots (slots beyond n_layer_ids are not written);
 * last_logits_host (optional) [vocab].  With feed_drafter every captured row is
 * appended to that drafter session, so n_layer_ids must equal the scratch's
 * capture slots. */
dfl_status dfl_prefill(const dfl_model* m, dfl_session* s, dfl_scratch* sc,
                       const uint32_t* layer_ids, uint32_t n_layer_ids, const int32_t* ids,
                       uint64_t n, uint32_t start_position, dfl_dsession* feed_drafter,
                       float* hidden_host, float* last_logits_host);

/* MetalDFlashSession::fresh(ctx, head, target_h, vocab, ctx_capacity)
 * metal_dflash.rs:5492. */
dfl_status dfl_dsession_create(const dfl_drafter* d, uint32_t ctx_capacity, dfl_dsession** out);
void dfl_dsession_destroy(dfl_dsession* ds);
uint32_t dfl_dsession_ctx_len(const dfl_dsession* ds);
/* append_target_ctx_columns_now  metal_dflash.rs:5798-5816: append `count`
 * columns of K*H f32 from the host (cols_host != NULL) ... */
dfl_status dfl_dsession_append_columns_host(dfl_dsession* ds, const float* cols_host,
                                            const uint32_t* positions, uint32_t count);
/* ... or rows [first_row, first_row+count) of the last verify capture. */
dfl_status dfl_dsession_append_from_scratch(dfl_dsession* ds, const dfl_scratch* sc,
                                            uint32_t first_row, uint32_t count,
                                            uint32_t first_position);
/* Drop all context columns (new request). */
dfl_status dfl_dsession_reset(dfl_dsession* ds);

/* DFlashDecoder::draft_block(carry, noise_start_pos) -> [N] tokens
 * metal_dflash.rs:15915; `_with_logits` :17499.  out_tokens[0] = carry,
 * out_tokens[1..N) = per-row argmax; logits_host optional [N * vocab]. */
dfl_status dfl_draft_block(dfl_dsession* ds, int32_t carry, uint32_t noise_start_pos,
                           int32_t* out_tokens, float* logits_host);
/* On a drafter with a DFlash 2 selector dfl_draft_block returns the selector's greedy path
 * (select_draft_path, metal_dflash.rs:17176-17251) instead of the per-row argmax. */

/* ---- DFlash 2 path selector ---------------------------------------------- */
/* kernel_topk16_f32 (kernels/dflash2.metal:96-170): per row the 16 best (id, value) pairs in
 * descending order under the f32 total order, ties to the lower index; rows shorter than 16
 * keep the sentinel (id -1, -inf) in the unfilled slots.  Host-to-host test entry. */
dfl_status dfl_topk16(int32_t device, const float* x_host, int32_t n_rows, uint64_t n,
                      int32_t* ids_out /* [n_rows][16] */, float* vals_out /* [n_rows][16] */);
/* DFlash2Codebook::from_gguf (metal_dflash.rs:3180-3273): host copy of a [rank, n_rows]
 * codebook, dtype Q4_K (rank 256 only) / Q8_0 / F32 / F16 / BF16. */
dfl_status dfl_codebook_create(int32_t dtype, uint64_t rank, uint64_t n_rows, const void* data,
                               uint64_t n_bytes, dfl_codebook** out);
void dfl_codebook_destroy(dfl_codebook* c);
/* DFlash2Codebook::dequant_row  metal_dflash.rs:3275-3340 */
dfl_status dfl_codebook_dequant_row(const dfl_codebook* c, uint64_t row, float* out, uint64_t n_out);
/* The greedy walk of select_draft_path (metal_dflash.rs:17212-17250) over ids / vals
 * [n][top_k] and the gate rows sel_h [n][rank]: tokens_out[0] = ids[0], tokens_out[pos] = the
 * candidate maximising vals + <A(prev) * sel_h[pos], B(candidate)> (strict >, first wins).
 * scores_out [n][top_k] and scored_out [n][top_k] (1 = candidate was scored) are optional
 * (diagnose_dflash2_selector_walk, metal_dflash.rs:3472-3620). */
dfl_status dfl_selector_walk(const dfl_codebook* predecessor, const dfl_codebook* successor,
                             uint32_t top_k, uint32_t rank, int32_t carry, uint32_t n,
                             const int32_t* ids, const float* vals, const float* sel_h,
                             int32_t* tokens_out, float* scores_out, uint8_t* scored_out);
/* The sampled walk of draft_block_sampled (metal_dflash.rs:17349-17409): each position's 16
 * scores are sampled with `proposal_sampler` (temperature only, else DFL_ERR_SAMPLING) and the
 * positive-weight candidates become that row's sparse proposal.  Row r = position r + 1 owns
 * candidates [cand_offsets[r], cand_offsets[r+1]); cand_offsets has n entries, cand_tokens /
 * cand_weights room for (n - 1) * top_k. */
dfl_status dfl_selector_walk_sampled(const dfl_codebook* predecessor, const dfl_codebook* successor,
                                     uint32_t top_k, uint32_t rank, int32_t carry, uint32_t n,
                                     const int32_t* ids, const float* vals, const float* sel_h,
                                     dfl_sampler* proposal_sampler, int32_t* tokens_out,
                                     uint32_t* cand_offsets, int32_t* cand_tokens,
                                     double* cand_weights);
/* DFlashDecoder::draft_block_sampled (metal_dflash.rs:17268-17415): one draft pass, then the
 * sampled walk.  Fails with DFL_ERR_UNSUPPORTED on a drafter without a selector ("sampled
 * path requires a DFlash 2 selector").  Outputs as dfl_selector_walk_sampled. */
dfl_status dfl_draft_block_sampled(dfl_dsession* ds, int32_t carry, uint32_t noise_start_pos,
                                   dfl_sampler* proposal_sampler, int32_t* out_tokens,
                                   uint32_t* cand_offsets, int32_t* cand_tokens,
                                   double* cand_weights);
/* Top-16 ids / logits [N][16] and, with a selector, the gate rows W_h h [N][rank] of the last
 * draft pass (the buffers draft_block_with_selector_diagnostic re-reads, metal_dflash.rs:17424).
 * sel_h_out may be NULL. */
dfl_status dfl_dsession_read_selector(dfl_dsession* ds, int32_t* ids_out, float* vals_out,
                                      float* sel_h_out);

/* ---- GGUF files (host) --------------------------------------------------- */
/* GgufFile::open (gguf.rs:154): maps a single-file GGUF (version 2 or 3), validates header, counts,
 * alignment and every tensor's extent against the file (gguf.rs:1094-1300).  Split files are refused. */
dfl_status dfl_gguf_open(const char* path, dfl_gguf** out);
void dfl_gguf_close(dfl_gguf* g);
uint64_t dfl_gguf_tensor_count(const dfl_gguf* g);
/* The file's tensors as one table, names and data pointing into the mapping (valid until close):
 * pass it to dfl_model_create as it is. */
const dfl_tensor* dfl_gguf_tensors(const dfl_gguf* g);
/* GgufFile::find (gguf.rs:474); DFL_ERR_MISSING_TENSOR when absent. */
dfl_status dfl_gguf_find(const dfl_gguf* g, const char* name, dfl_tensor* out);
/* Typed metadata getters (gguf.rs:514-729).  *found = 0 when the key is absent (or, for u64 / f64 /
 * str, of another type); get_bool and the array getter fail when the key exists with a wrong type. */
dfl_status dfl_gguf_get_u64(const dfl_gguf* g, const char* key, uint64_t* out, int32_t* found);
dfl_status dfl_gguf_get_f64(const dfl_gguf* g, const char* key, double* out, int32_t* found);
dfl_status dfl_gguf_get_bool(const dfl_gguf* g, const char* key, int32_t* out, int32_t* found);
dfl_status dfl_gguf_get_str(const dfl_gguf* g, const char* key, char* buf, uint64_t cap, int32_t* found);
/* integer or bool arrays widened to u64; out may be NULL to query *count */
dfl_status dfl_gguf_get_u64_array(const dfl_gguf* g, const char* key, uint64_t* out, uint64_t cap,
                                  uint64_t* count, int32_t* found);
/* build_arch_from_metadata (loader.rs:1331-1656): `qwen35.*` / `qwen35moe.*` keys -> dfl_arch. */
dfl_status dfl_gguf_arch(const dfl_gguf* g, dfl_arch* out);
/* The drafter's DFlashConfig (loader.rs:860-1060) from a "dflash-draft" or "dflash" file. */
dfl_status dfl_gguf_dflash_config(const dfl_gguf* drafter, const dfl_arch* target, dfl_dflash_config* out);
/* The drafter file's tensors under the names dfl_drafter_create expects (the "dflash" format's
 * fc / enc.output_norm / ffn_norm names mapped to the "dflash-draft" ones, loader.rs:876-912). */
dfl_status dfl_gguf_drafter_tensors(dfl_gguf* g, const dfl_tensor** table, uint64_t* count);

/* ---- sampling + acceptance (host, f64) --------------------------------- */
typedef struct dfl_sampling_config { /* SamplingConfig  sampling.rs:17-30 */
    float temperature;
    uint32_t top_k;
    float top_p;
    float min_p;
    uint64_t seed;
} dfl_sampling_config;

dfl_status dfl_sampler_create(const dfl_sampling_config* cfg, dfl_sampler** out);
/* Sampler::at_draw  sampling.rs:359 */
dfl_status dfl_sampler_create_at_draw(const dfl_sampling_config* cfg, uint64_t draws,
                                      dfl_sampler** out);
void dfl_sampler_destroy(dfl_sampler* s);
/* Sampler::config  sampling.rs:369 */
void dfl_sampler_get_config(const dfl_sampler* s, dfl_sampling_config* out);
uint64_t dfl_sampler_draws(const dfl_sampler* s);
void dfl_sampler_rng_state(const dfl_sampler* s, uint64_t out_state[4]);
/* Presorted rows.  The sampler orders a row's candidates by descending logit (total order, ties by ascending
 * token: sampling.rs:305-790) before anything else; that order is a pure function of the logits' bits, and the device
 * can produce it (dfl_scratch_set_order_host).  After this call, a row whose logits pointer is
 * logits_base + r * vocab (r < n_rows) takes its order from order_base + r * vocab instead of sorting; an order that
 * is not the row's sorted order is detected and ignored (the row is then sorted on the host).  NULL bases clear the
 * registration.  The caller keeps both arrays alive while registered. */
dfl_status dfl_sampler_set_row_order(dfl_sampler* s, const float* logits_base, const uint32_t* order_base,
                                     uint32_t n_rows, uint64_t vocab);
/* Host threads dfl_accept_prefix may use to build a block's row distributions ahead of its sequential loop (the picks
 * stay sequential, so nothing drawn or decided changes): 0 = as many as the host reports, 1 = none - every row is built
 * by the calling thread when the loop reaches it, which is the right choice when every core already drives a sequence -
 * n > 1 = at most n. */
dfl_status dfl_sampler_set_worker_threads(dfl_sampler* s, uint32_t n);
/* Rows that took a registered order since the sampler was created (rows whose order was refused are not counted). */
uint64_t dfl_sampler_preordered_rows(const dfl_sampler* s);
/* Sampler::sample  sampling.rs:530 */
dfl_status dfl_sampler_sample(dfl_sampler* s, const float* logits, uint64_t vocab,
                              int32_t* token_out, uint64_t* candidate_index_out);
/* Sampler::sample_with_distribution  sampling.rs:437-452: samples and also returns the
 * filtered categorical distribution (tokens / unnormalised weights in categorical order,
 * at most `cap` entries; *count receives the full length). */
dfl_status dfl_sampler_sample_with_distribution(dfl_sampler* s, const float* logits, uint64_t vocab,
                                                int32_t* token_out, uint64_t* candidate_index_out,
                                                int32_t* dist_tokens, double* dist_weights,
                                                uint64_t cap, uint64_t* count, double* total_weight);
/* greedy_token  sampling.rs:1159-1181 */
dfl_status dfl_greedy_token(const float* logits, uint64_t vocab, int32_t* token_out);
/* raw generator access for golden-vector checks (sampling.rs:1621-1670) */
uint64_t dfl_splitmix64_next(uint64_t* state);
uint64_t dfl_sampler_next_u64(dfl_sampler* s);
double dfl_sampler_next_unit_f64(dfl_sampler* s);

/* SparseProposal rows, flattened: row r owns candidates
 * [cand_offsets[r], cand_offsets[r+1]).  sampling.rs:185-197. */
typedef struct dfl_sparse_proposals {
    uint32_t n_rows;
    const int32_t* tokens;        /* [n_rows] sampled proposal token per row */
    const uint32_t* cand_offsets; /* [n_rows + 1] */
    const int32_t* cand_tokens;
    const double* cand_weights;
} dfl_sparse_proposals;

enum { DFL_CARRY_NONE = 0, DFL_CARRY_CORRECTION = 1, DFL_CARRY_BONUS = 2 };
enum { DFL_STOP_NONE = 0, DFL_STOP_EOS = 1, DFL_STOP_TOKEN_LIMIT = 2 };

typedef struct dfl_accept_decision { /* DFlashAcceptDecision  accept.rs:17-32 */
    uint32_t n_accepted;
    int32_t accepted_drafts[DFL_MAX_BLOCK];
    int32_t next_carry_kind;
    int32_t next_carry;
    int32_t stop_reason;
    uint32_t retain_input_count;
    int32_t error_row; /* row of a Sampling error, else -1 */
} dfl_accept_decision;

/* decide_dflash_accept_prefix  metal_dflash/accept.rs:76-183.  On any error the
 * sampler is left unchanged. */
dfl_status dfl_accept_prefix(const int32_t* verified_tokens, uint32_t n_tokens,
                             const float* target_logits, uint64_t n_logits, uint64_t vocab,
                             const dfl_sparse_proposals* proposals /* NULL = deterministic */,
                             dfl_sampler* sampler, uint64_t remaining_output_budget,
                             const int32_t* stop_ids, uint32_t n_stop_ids,
                             dfl_accept_decision* out);
/* Sampler::couple_sparse_proposal  sampling.rs:708-790; decision 1 = accepted,
 * 0 = rejected with *correction set. */
dfl_status dfl_sampler_couple_sparse(dfl_sampler* s, const float* logits, uint64_t vocab,
                                     int32_t proposal_token, const int32_t* cand_tokens,
                                     const double* cand_weights, uint32_t n_cand,
                                     int32_t* accepted, int32_t* correction);

/* ---- the outer loop ----------------------------------------------------- */
typedef struct dfl_generate_params {
    uint32_t max_tokens;
    const int32_t* stop_ids;
    uint32_t n_stop_ids;
    /* "replayed drafts" (dflash_prefix_replay_drafts, qwen/dflash.rs:351-376):
     * when non-NULL the drafter is bypassed and drafts are taken from this
     * history wherever it agrees with what was emitted. */
    const int32_t* replay_history;
    uint32_t n_replay_history;
    /* sampled mode: build sparse proposals from the drafter's top-16
     * (draft_block_sampled, metal_dflash.rs:17268-17415) instead of one-hot. */
    int32_t sparse_proposals;
    /* margin guard (qwen/dflash.rs:93-121): committed rows with gap < margin are counted (stats.margin_rows, and
     * stats.fallback_steps for the steps that hold one).  The reference replays such rows through its exact
     * single-token path; here a packed row and a single-token row are the same bits, so the replay would reproduce
     * the row and is not run.  0 disables. */
    float verify_margin;
    /* with replay_history: still run the drafter every step (its tokens are discarded) so that a
     * replayed-acceptance schedule pays the full draft cost. */
    int32_t replay_runs_drafter;
    /* with replay_history: take drafts from history[emitted ...] even where the history disagrees
     * with what was emitted (the reference stops replaying at the first divergence).  Lets a caller
     * script an acceptance schedule by corrupting chosen draft positions. */
    int32_t replay_unchecked;
    /* sampled mode: order every verify row on the device (dfl_scratch_set_order_host) and hand the order to the
     * sampler (dfl_sampler_set_row_order), which then skips its own ordering of the 151 936-token rows.  Draws,
     * decisions and generator state are unchanged. */
    int32_t device_row_order;
} dfl_generate_params;

typedef struct dfl_generate_stats { /* DflashDecodeStats  qwen/dflash.rs:380-418 */
    uint32_t spec_steps;
    uint32_t drafter_calls;
    uint32_t verify_calls;
    uint32_t restore_calls;
    uint32_t fallback_steps;
    uint64_t drafts_scored;
    uint64_t accepted_drafts;
    uint64_t tokens_emitted;
    double draft_ms;    /* device time, CUDA events */
    double verify_ms;
    double restore_ms;
    double accept_ms;   /* host */
    double append_ms;
    double wall_ms;
    /* margin guard accounting (greedy mode, verify_margin > 0): committed verify rows, and how many of them had a
     * top-1 / top-2 gap below the margin (qwen/dflash.rs:93-121 counts the same rows before replaying them) */
    uint64_t committed_rows;
    uint64_t margin_rows;
} dfl_generate_stats;

/* generate_dflash  crates/qwen-cli/src/qwen/dflash.rs:484-1263.  `first_logits`
 * [vocab] are the logits of the last prompt position; tokens_out has room for
 * max_tokens ids; *n_out receives the count. */
dfl_status dfl_generate(const dfl_model* m, dfl_session* s, dfl_scratch* sc, dfl_dsession* ds,
                        dfl_sampler* sampler, const float* first_logits,
                        const dfl_generate_params* params, int32_t* tokens_out, uint32_t* n_out,
                        dfl_generate_stats* stats);

/* ---- synthetic weights (no reference counterpart: the reference loads GGUF
 * files; benchmarks here use seeded N(0, std) weights quantised on the GPU) -- */
/* Fills a device buffer with a [n_out][n_in] tensor of `dtype` in ggml block
 * layout from a counter-based generator; *dev_ptr must be freed with
 * dfl_device_free. */
dfl_status dfl_synth_tensor(int32_t device, int32_t dtype, uint64_t n_in, uint64_t n_out,
                            uint64_t seed, float std_dev, void** dev_ptr, uint64_t* n_bytes);
dfl_status dfl_device_free(int32_t device, void* dev_ptr);
dfl_status dfl_device_to_host(int32_t device, const void* dev_ptr, void* host, uint64_t n_bytes);

#ifdef __cplusplus
}
#endif
#endif /* DFLASH_B200_H */
