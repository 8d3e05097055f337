"""Host-side Python mirror of the dflash_b200 C ABI (include/dflash_b200.h).

The package is a thin ctypes layer: every call goes through the `extern "C"` entry
points of libdflash_b200.so, the same ones a Rust/cgo/JNI binding would use.  There is
no CPU fallback: if the CUDA library has not been built, importing a compute symbol
raises; if no GPU is present the library returns DFL_ERR_NO_DEVICE.
"""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libdflash_b200.so")

F32, F16, Q8_0, Q4_K, Q5_K, Q6_K, BF16 = 0, 1, 8, 12, 13, 14, 30
MAX_BLOCK = 16
MAX_TARGET_LAYERS = 8
MAX_DRAFTER_LAYERS = 16

STATUS_NAMES = {0: "OK", 1: "BAD_ARG", 2: "BAD_SHAPE", 3: "UNSUPPORTED", 4: "CUDA", 5: "NO_DEVICE", 6: "OOM", 7: "POISONED",
                8: "CTX_OVERFLOW", 9: "KV_STATE", 10: "BAD_TOKEN", 11: "SAMPLING", 12: "TIMEOUT", 13: "MISSING_TENSOR", 14: "ROUTE_STATUS", 15: "COLLECTIVE"}


class DflError(RuntimeError):
    def __init__(self, status, message):
        super().__init__(f"DFL_ERR_{STATUS_NAMES.get(status, status)}: {message}")
        self.status = status
        self.name = STATUS_NAMES.get(status, str(status))


class Tensor(C.Structure):
    _fields_ = [("name", C.c_char_p), ("dtype", C.c_int32), ("n_dims", C.c_int32), ("shape", C.c_uint64 * 4),
                ("data", C.c_void_p), ("n_bytes", C.c_uint64), ("on_device", C.c_int32), ("_pad", C.c_int32)]


class Arch(C.Structure):
    _fields_ = [("n_layer", C.c_uint32), ("hidden_size", C.c_uint32), ("intermediate_size", C.c_uint32),
                ("vocab_size", C.c_uint32), ("full_attention_interval", C.c_uint32), ("n_q_heads", C.c_uint32),
                ("n_kv_heads", C.c_uint32), ("attn_head_dim", C.c_uint32), ("rope_theta", C.c_float),
                ("partial_rotary_factor", C.c_float), ("gdn_n_v_heads", C.c_uint32), ("gdn_n_k_heads", C.c_uint32),
                ("gdn_head_dim", C.c_uint32), ("gdn_conv_kernel", C.c_uint32), ("expert_count", C.c_uint32),
                ("expert_used_count", C.c_uint32), ("expert_feed_forward_length", C.c_uint32),
                ("expert_shared_feed_forward_length", C.c_uint32)]


class DFlashConfig(C.Structure):
    _fields_ = [("n_layer", C.c_uint32), ("hidden_size", C.c_uint32), ("intermediate_size", C.c_uint32),
                ("n_q_heads", C.c_uint32), ("n_kv_heads", C.c_uint32), ("head_dim", C.c_uint32), ("rope_theta", C.c_float),
                ("rms_norm_eps", C.c_float), ("causal", C.c_uint32), ("swa_window", C.c_uint32), ("block_size", C.c_uint32),
                ("mask_token_id", C.c_int32), ("n_target_layers", C.c_uint32),
                ("target_layer_ids", C.c_uint32 * MAX_TARGET_LAYERS), ("layer_is_swa", C.c_uint32 * MAX_DRAFTER_LAYERS),
                ("selector_rank", C.c_uint32), ("selector_top_k", C.c_uint32)]


class SamplingConfig(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_k", C.c_uint32), ("top_p", C.c_float), ("min_p", C.c_float),
                ("seed", C.c_uint64)]


class SparseProposals(C.Structure):
    _fields_ = [("n_rows", C.c_uint32), ("tokens", C.POINTER(C.c_int32)), ("cand_offsets", C.POINTER(C.c_uint32)),
                ("cand_tokens", C.POINTER(C.c_int32)), ("cand_weights", C.POINTER(C.c_double))]


class AcceptDecision(C.Structure):
    _fields_ = [("n_accepted", C.c_uint32), ("accepted_drafts", C.c_int32 * MAX_BLOCK), ("next_carry_kind", C.c_int32),
                ("next_carry", C.c_int32), ("stop_reason", C.c_int32), ("retain_input_count", C.c_uint32),
                ("error_row", C.c_int32)]


class GenerateParams(C.Structure):
    _fields_ = [("max_tokens", C.c_uint32), ("stop_ids", C.POINTER(C.c_int32)), ("n_stop_ids", C.c_uint32),
                ("replay_history", C.POINTER(C.c_int32)), ("n_replay_history", C.c_uint32), ("sparse_proposals", C.c_int32),
                ("verify_margin", C.c_float), ("replay_runs_drafter", C.c_int32), ("replay_unchecked", C.c_int32),
                ("device_row_order", C.c_int32)]


class GenerateStats(C.Structure):
    _fields_ = [("spec_steps", C.c_uint32), ("drafter_calls", C.c_uint32), ("verify_calls", C.c_uint32),
                ("restore_calls", C.c_uint32), ("fallback_steps", C.c_uint32), ("drafts_scored", C.c_uint64),
                ("accepted_drafts", C.c_uint64), ("tokens_emitted", C.c_uint64), ("draft_ms", C.c_double),
                ("verify_ms", C.c_double), ("restore_ms", C.c_double), ("accept_ms", C.c_double), ("append_ms", C.c_double),
                ("wall_ms", C.c_double), ("committed_rows", C.c_uint64), ("margin_rows", C.c_uint64)]


_LIB = None


def lib():
    """The loaded C ABI.  Raises if the CUDA library was not built (no fallback)."""
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: run `python qwen-llm_b200/build.py` (needs nvcc). "
                              "There is no CPU implementation to fall back to.")
        L = C.CDLL(LIB_PATH)
        L.dfl_version.restype = C.c_char_p
        L.dfl_last_error.restype = C.c_char_p
        L.dfl_device_count.restype = C.c_int32
        L.dfl_launch_count.restype = C.c_uint64
        for name in ("dfl_model_verify_weight_bytes", "dfl_model_verify_resident_bytes", "dfl_drafter_weight_bytes", "dfl_sampler_draws", "dfl_sampler_preordered_rows",
                     "dfl_splitmix64_next", "dfl_sampler_next_u64"):
            if hasattr(L, name):
                getattr(L, name).restype = C.c_uint64
        for name in ("dfl_session_kv_n_pos", "dfl_dsession_ctx_len"):
            if hasattr(L, name):
                getattr(L, name).restype = C.c_uint32
        if hasattr(L, "dfl_gguf_tensors"):
            L.dfl_gguf_tensors.restype = C.POINTER(Tensor)
            L.dfl_gguf_tensor_count.restype = C.c_uint64
        if hasattr(L, "dfl_sampler_next_unit_f64"):
            L.dfl_sampler_next_unit_f64.restype = C.c_double
        _LIB = L
    return _LIB


def check(status):
    if status != 0:
        raise DflError(status, lib().dfl_last_error().decode(errors="replace"))


def _ptr(a, t=C.c_void_p):
    return a.ctypes.data_as(t)


def set_host_wait(mode):
    """'auto' | 'spin' | 'yield' | 'block': how host threads wait for the device (dfl_set_host_wait)."""
    check(lib().dfl_set_host_wait(C.c_int32({"auto": 0, "spin": 1, "yield": 2, "block": 3}[mode])))


def device_count():
    return int(lib().dfl_device_count())


def launch_count():
    return int(lib().dfl_launch_count())


class QMatrix:
    """A resident quantised matrix W[n_out][n_in] (ggml bytes in, stream tiles on the GPU)."""

    def __init__(self, dtype, n_in, n_out, raw, device=0):
        raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
        self.dtype, self.n_in, self.n_out, self.device = dtype, n_in, n_out, device
        self.h = C.c_void_p()
        check(lib().dfl_qmatrix_create(C.c_int32(device), C.c_int32(dtype), C.c_uint64(n_in), C.c_uint64(n_out), _ptr(raw),
                                       C.c_uint64(raw.size), C.c_int32(0), C.byref(self.h)))

    def close(self):
        if self.h:
            lib().dfl_qmatrix_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def engine(self):
        """'tcgen05' | 'mma.sync' | 'f32' (dfl_qmatrix_engine)."""
        return {2: "tcgen05", 1: "mma.sync", 0: "f32"}[int(lib().dfl_qmatrix_engine(self.h))]

    def dequant(self):
        out = np.zeros((self.n_out, self.n_in), dtype=np.float32)
        check(lib().dfl_qmatrix_dequant(self.h, _ptr(out), C.c_uint64(out.size)))
        return out

    def matmul(self, x):
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, self.n_in)
        y = np.zeros((x.shape[0], self.n_out), dtype=np.float32)
        check(lib().dfl_fewrow_matmul(self.h, _ptr(x), C.c_int32(x.shape[0]), _ptr(y)))
        return y


def argmax_top2(logits, device=0):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    n, v = logits.shape
    am = np.zeros(n, dtype=np.int32)
    gap = np.zeros(n, dtype=np.float32)
    check(lib().dfl_argmax_top2(C.c_int32(device), _ptr(logits), C.c_int32(n), C.c_uint64(v), _ptr(am), _ptr(gap)))
    return am, gap


def argmax_top2_static(logits_ptr, n_rows, vocab, ld, argmax_ptr, gap_ptr, stream=0, device=0):
    """Row argmax over device buffers given as raw addresses; enqueues on `stream` and allocates nothing."""
    check(lib().dfl_argmax_top2_static(C.c_int32(device), C.c_void_p(logits_ptr), C.c_int32(n_rows), C.c_uint64(vocab),
                                       C.c_uint64(ld), C.c_void_p(argmax_ptr), C.c_void_p(gap_ptr), C.c_void_p(stream)))


class C1Pipeline:
    """The CPU-runnable verify / accept case: logits = head(x W1^T), row argmax, greedy prefix acceptance."""

    def __init__(self, w1: QMatrix, head: QMatrix):
        self.w1, self.head = w1, head
        self.h = C.c_void_p()
        check(lib().dfl_c1_create(w1.h, head.h, C.byref(self.h)))

    def close(self):
        if self.h:
            lib().dfl_c1_destroy(self.h)
            self.h = C.c_void_p()

    def step(self, x, draft_ids, want_logits=False):
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, self.w1.n_in)
        n = x.shape[0]
        draft = np.ascontiguousarray(draft_ids, dtype=np.int32)
        am = np.zeros(n, dtype=np.int32)
        gap = np.zeros(n, dtype=np.float32)
        nacc = C.c_int32(0)
        logits = np.zeros((n, self.head.n_out), dtype=np.float32) if want_logits else None
        check(lib().dfl_c1_step(self.h, _ptr(x), C.c_int32(n), _ptr(draft), _ptr(am), _ptr(gap), C.byref(nacc),
                                _ptr(logits) if want_logits else None))
        return am, gap, int(nacc.value), logits

    def upload(self, x):
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, self.w1.n_in)
        check(lib().dfl_c1_upload(self.h, _ptr(x), C.c_int32(x.shape[0])))

    def run_resident(self, n_rows, iters):
        ms = C.c_float(0)
        check(lib().dfl_c1_run_resident(self.h, C.c_int32(n_rows), C.c_int32(iters), C.byref(ms)))
        return float(ms.value)


# ---------------------------------------------------------------------------
# model / session / scratch
# ---------------------------------------------------------------------------
def make_tensor_table(tensors):
    """tensors: list of (name, dtype, shape(list, ne[0] first), numpy uint8 bytes). Returns (ctypes array, keepalive)."""
    arr = (Tensor * len(tensors))()
    keep = []
    for i, (name, dtype, shape, raw) in enumerate(tensors):
        raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
        nm = name.encode()
        keep.append((nm, raw))
        arr[i].name = nm
        arr[i].dtype = dtype
        arr[i].n_dims = len(shape)
        for j, d in enumerate(shape):
            arr[i].shape[j] = d
        arr[i].data = raw.ctypes.data
        arr[i].n_bytes = raw.size
        arr[i].on_device = 0
    return arr, keep


def ep_unique_id():
    """128-byte NCCL id (call on one rank, hand to every rank of the expert-parallel group)."""
    buf = (C.c_uint8 * 128)()
    check(lib().dfl_ep_unique_id(buf))
    return bytes(buf)


def ep_watchdog_selftest(scenario, after_polls=3, timeout_ms=200):
    """Drives the expert-parallel host watchdog's polling loop with scripted actions (no GPU).  Returns how often the
    abort action ran; raises DflError COLLECTIVE when the loop gave up (scenarios 1-3)."""
    aborted = C.c_int32(-1)
    st = lib().dfl_ep_watchdog_selftest(C.c_int32(scenario), C.c_uint32(after_polls), C.c_uint32(timeout_ms), C.byref(aborted))
    if st != 0:
        err = DflError(st, lib().dfl_last_error().decode(errors="replace"))
        err.aborted = aborted.value
        raise err
    return aborted.value


class Model:
    def __init__(self, arch: Arch, tensors, device=0, ep=None):
        """ep = (rank, world, nccl_id) builds the expert-parallel slice of a routed-expert model."""
        arr, keep = make_tensor_table(tensors)
        self.arch, self.device = arch, device
        self.h = C.c_void_p()
        if ep is None:
            check(lib().dfl_model_create(C.c_int32(device), C.byref(arch), arr, C.c_uint64(len(tensors)), C.byref(self.h)))
        else:
            rank, world, nccl_id = ep
            idb = (C.c_uint8 * 128).from_buffer_copy(nccl_id)
            check(lib().dfl_model_create_ep(C.c_int32(device), C.byref(arch), arr, C.c_uint64(len(tensors)), C.c_int32(rank),
                                            C.c_int32(world), idb, C.byref(self.h)))

    @classmethod
    def from_gguf(cls, gguf, device=0):
        """Builds the target from an open GGUF: arch from its metadata, weights from its tensor table."""
        self = cls.__new__(cls)
        self.arch, self.device = gguf.arch(), device
        self.h = C.c_void_p()
        tab, n = gguf.table()
        check(lib().dfl_model_create(C.c_int32(device), C.byref(self.arch), tab, C.c_uint64(n), C.byref(self.h)))
        return self

    def verify_weight_bytes(self):
        return int(lib().dfl_model_verify_weight_bytes(self.h))

    def verify_resident_bytes(self):
        return int(lib().dfl_model_verify_resident_bytes(self.h))

    def close(self):
        if self.h:
            lib().dfl_model_destroy(self.h)
            self.h = C.c_void_p()


class Session:
    def __init__(self, model: Model, kv_capacity, kv_f16=True):
        self.model = model
        self.h = C.c_void_p()
        check(lib().dfl_session_create(model.h, C.c_uint32(kv_capacity), C.c_int32(1 if kv_f16 else 0), C.byref(self.h)))

    @property
    def kv_n_pos(self):
        return int(lib().dfl_session_kv_n_pos(self.h))

    @property
    def poisoned(self):
        return bool(lib().dfl_session_poisoned(self.h))

    def fail_next_completion(self):
        lib().dfl_session_fail_next_completion(self.h)

    def probe_wait_timeout(self, polls=256):
        """Runs the wait probe (a bounded device-side wait that nothing satisfies); raises DflError TIMEOUT."""
        check(lib().dfl_session_probe_wait_timeout(self.model.h, self.h, C.c_uint32(polls)))

    def read_gdn_state(self, gdn_index):
        a = self.model.arch
        ssm = np.zeros(a.gdn_n_v_heads * 128 * 128, dtype=np.float32)
        conv = np.zeros(3 * (2 * a.gdn_n_k_heads + a.gdn_n_v_heads) * 128, dtype=np.float32)
        check(lib().dfl_session_read_gdn_state(self.h, C.c_uint32(gdn_index), _ptr(ssm), C.c_uint64(ssm.size), _ptr(conv),
                                               C.c_uint64(conv.size)))
        return ssm, conv

    def read_kv(self, attn_index, pos):
        a = self.model.arch
        n = a.n_kv_heads * a.attn_head_dim
        k = np.zeros(n, dtype=np.float32)
        v = np.zeros(n, dtype=np.float32)
        check(lib().dfl_session_read_kv(self.h, C.c_uint32(attn_index), C.c_uint32(pos), _ptr(k), _ptr(v), C.c_uint64(n)))
        return k, v

    def close(self):
        if self.h:
            lib().dfl_session_destroy(self.h)
            self.h = C.c_void_p()


class Scratch:
    def __init__(self, model: Model, block_size=16, n_capture_layers=0):
        self.model, self.block_size, self.k = model, block_size, max(1, n_capture_layers)
        self.h = C.c_void_p()
        check(lib().dfl_scratch_create(model.h, C.c_uint32(block_size), C.c_uint32(n_capture_layers), C.byref(self.h)))

    def read_capture(self, n):
        out = np.zeros((n, self.k, self.model.arch.hidden_size), dtype=np.float32)
        check(lib().dfl_scratch_read_capture(self.h, C.c_uint32(n), _ptr(out), C.c_uint64(out.size)))
        return out

    def read_route(self, n):
        """Expert ids [n][expert_used_count] the last routed-expert layer of the last verify chose."""
        out = np.zeros((n, self.model.arch.expert_used_count), dtype=np.int32)
        check(lib().dfl_scratch_read_route(self.h, C.c_uint32(n), _ptr(out), C.c_uint64(out.size)))
        return out

    def close(self):
        if self.h:
            lib().dfl_scratch_destroy(self.h)
            self.h = C.c_void_p()


def _u32(a):
    return np.ascontiguousarray(a, dtype=np.uint32)


def packed_verify(model, session, scratch, layer_ids, tokens, start_position, want_logits=False, want_order=False):
    """want_order (with want_logits): also returns each row's token ids by descending logit, ordered on the device."""
    tokens = np.ascontiguousarray(tokens, dtype=np.int32)
    n = tokens.size
    ids = _u32(layer_ids)
    am = np.zeros(n, dtype=np.int32)
    gap = np.zeros(n, dtype=np.float32)
    logits = np.zeros((n, model.arch.vocab_size), dtype=np.float32) if want_logits else None
    if want_order:
        order = np.zeros((scratch.block_size, model.arch.vocab_size), dtype=np.uint32)
        check(lib().dfl_scratch_set_order_host(scratch.h, _ptr(order, C.POINTER(C.c_uint32))))
        try:
            check(lib().dfl_packed_verify(model.h, session.h, scratch.h, _ptr(ids) if ids.size else None, C.c_uint32(ids.size),
                                          _ptr(tokens), C.c_uint32(n), C.c_uint32(start_position), _ptr(am), _ptr(gap), _ptr(logits)))
        finally:
            lib().dfl_scratch_set_order_host(scratch.h, None)
        return am, gap, logits, order[:n]
    check(lib().dfl_packed_verify(model.h, session.h, scratch.h, _ptr(ids) if ids.size else None, C.c_uint32(ids.size), _ptr(tokens),
                                  C.c_uint32(n), C.c_uint32(start_position), _ptr(am), _ptr(gap),
                                  _ptr(logits) if want_logits else None))
    return am, gap, logits


def packed_verify_n_eff(model, session, scratch, layer_ids, tokens, start_position, n_eff_override=None):
    """packed_verify with the reference's n_eff_override argument (None = the scratch's block size)."""
    tokens = np.ascontiguousarray(tokens, dtype=np.int32)
    ids = _u32(layer_ids)
    am = np.zeros(max(tokens.size, 1), dtype=np.int32)
    gap = np.zeros(max(tokens.size, 1), dtype=np.float32)
    check(lib().dfl_packed_verify_n_eff(model.h, session.h, scratch.h, _ptr(ids) if ids.size else None, C.c_uint32(ids.size), _ptr(tokens),
                                        C.c_uint32(tokens.size), C.c_uint32(start_position),
                                        C.c_int32(-1 if n_eff_override is None else n_eff_override), _ptr(am), _ptr(gap), None))
    return am[:tokens.size], gap[:tokens.size]


def restore_partial_n_eff(model, session, scratch, n_keep, start_position, n_eff_override=None):
    check(lib().dfl_restore_partial_n_eff(model.h, session.h, scratch.h, C.c_uint32(n_keep), C.c_uint32(start_position),
                                          C.c_int32(-1 if n_eff_override is None else n_eff_override)))


class SnapshotIdentity(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("layout_version", "n_attn_layers", "n_gdn_layers", "kv_dim_elements", "kv_bytes_per_token",
                                          "kv_storage_kind", "gdn_state_elements_per_layer", "gdn_conv_elements_per_layer")]


def snapshot_identity(model, session):
    out = SnapshotIdentity()
    check(lib().dfl_session_snapshot_identity(model.h, session.h, C.byref(out)))
    return out


def session_snapshot(model, session, dsession=None):
    """SessionSnapshot of the current prefix (and the drafter's visible context) as one byte array."""
    lib().dfl_session_snapshot_bytes.restype = C.c_uint64
    n = int(lib().dfl_session_snapshot_bytes(model.h, session.h, dsession.h if dsession is not None else None))
    blob = np.zeros(n, dtype=np.uint8)
    written = C.c_uint64(0)
    check(lib().dfl_session_snapshot(model.h, session.h, dsession.h if dsession is not None else None, _ptr(blob), C.c_uint64(n), C.byref(written)))
    return blob[:int(written.value)]


def session_restore_snapshot(model, session, dsession, blob):
    blob = np.ascontiguousarray(blob, dtype=np.uint8)
    check(lib().dfl_session_restore_snapshot(model.h, session.h, dsession.h if dsession is not None else None, _ptr(blob), C.c_uint64(blob.size)))


def restore_partial(model, session, scratch, n_keep, start_position):
    check(lib().dfl_restore_partial(model.h, session.h, scratch.h, C.c_uint32(n_keep), C.c_uint32(start_position)))


def restore_pre_block(model, session, scratch, start_position):
    check(lib().dfl_restore_pre_block(model.h, session.h, scratch.h, C.c_uint32(start_position)))


def single_token(model, session, scratch, layer_ids, token, position, want_hidden=True):
    ids = _u32(layer_ids)
    logits = np.zeros(model.arch.vocab_size, dtype=np.float32)
    hidden = np.zeros((ids.size, model.arch.hidden_size), dtype=np.float32) if (want_hidden and ids.size) else None
    check(lib().dfl_single_token(model.h, session.h, scratch.h, _ptr(ids) if ids.size else None, C.c_uint32(ids.size),
                                 C.c_int32(int(token)), C.c_uint32(position), _ptr(logits),
                                 _ptr(hidden) if hidden is not None else None))
    return logits, hidden


# ---------------------------------------------------------------------------
# sampler + acceptance (host)
# ---------------------------------------------------------------------------
class Sampler:
    def __init__(self, temperature=0.0, top_k=0, top_p=1.0, min_p=0.0, seed=0, at_draw=None):
        self.cfg = SamplingConfig(temperature, top_k, top_p, min_p, seed & ((1 << 64) - 1))
        self.h = C.c_void_p()
        if at_draw is None:
            check(lib().dfl_sampler_create(C.byref(self.cfg), C.byref(self.h)))
        else:
            check(lib().dfl_sampler_create_at_draw(C.byref(self.cfg), C.c_uint64(at_draw), C.byref(self.h)))

    def close(self):
        if self.h:
            lib().dfl_sampler_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def draws(self):
        return int(lib().dfl_sampler_draws(self.h))

    def set_worker_threads(self, n):
        """0: as many row-building threads as the host reports; 1: none (rows built on demand); n: at most n."""
        check(lib().dfl_sampler_set_worker_threads(self.h, C.c_uint32(n)))

    @property
    def preordered_rows(self):
        return int(lib().dfl_sampler_preordered_rows(self.h))

    def rng_state(self):
        st = (C.c_uint64 * 4)()
        lib().dfl_sampler_rng_state(self.h, st)
        return list(st)

    def next_u64(self):
        return int(lib().dfl_sampler_next_u64(self.h))

    def next_unit_f64(self):
        return float(lib().dfl_sampler_next_unit_f64(self.h))

    def set_row_order(self, logits, order):
        """Registers presorted rows: `order` [n][vocab] u32 for the C-contiguous f32 `logits` [n][vocab] (both kept alive
        by this object and passed to sample() / accept_prefix() as views of these very arrays); None clears."""
        self._row_order_keep = None
        if logits is None or order is None:
            check(lib().dfl_sampler_set_row_order(self.h, None, None, C.c_uint32(0), C.c_uint64(0)))
            return
        assert logits.dtype == np.float32 and order.dtype == np.uint32 and logits.flags.c_contiguous and order.flags.c_contiguous
        assert logits.shape == order.shape and logits.ndim == 2
        check(lib().dfl_sampler_set_row_order(self.h, _ptr(logits), _ptr(order, C.POINTER(C.c_uint32)), C.c_uint32(logits.shape[0]),
                                              C.c_uint64(logits.shape[1])))
        self._row_order_keep = (logits, order)   # the library reads both arrays until the registration is cleared

    def sample(self, logits):
        logits = np.ascontiguousarray(logits, dtype=np.float32)
        tok, idx = C.c_int32(0), C.c_uint64(0)
        check(lib().dfl_sampler_sample(self.h, _ptr(logits), C.c_uint64(logits.size), C.byref(tok), C.byref(idx)))
        return int(tok.value), int(idx.value)

    def couple_sparse(self, logits, token, candidates):
        logits = np.ascontiguousarray(logits, dtype=np.float32)
        ct = np.ascontiguousarray([c[0] for c in candidates], dtype=np.int32)
        cw = np.ascontiguousarray([c[1] for c in candidates], dtype=np.float64)
        acc, corr = C.c_int32(0), C.c_int32(0)
        check(lib().dfl_sampler_couple_sparse(self.h, _ptr(logits), C.c_uint64(logits.size), C.c_int32(token), _ptr(ct), _ptr(cw),
                                              C.c_uint32(ct.size), C.byref(acc), C.byref(corr)))
        return ("accepted", None) if acc.value else ("rejected", int(corr.value))


def topk16(x, device=0):
    """kernel_topk16_f32 on the device: ids, vals [n_rows][16]."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    ids = np.zeros((x.shape[0], 16), dtype=np.int32)
    vals = np.zeros((x.shape[0], 16), dtype=np.float32)
    check(lib().dfl_topk16(C.c_int32(device), _ptr(x), C.c_int32(x.shape[0]), C.c_uint64(x.shape[1]), _ptr(ids), _ptr(vals)))
    return ids, vals


def sort_rows_desc(x, device=0):
    """Token ids of every row by descending value (f32 total order, ties by ascending index), ordered on the device."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    order = np.zeros(x.shape, dtype=np.uint32)
    check(lib().dfl_sort_rows_desc(C.c_int32(device), _ptr(x), C.c_int32(x.shape[0]), C.c_uint64(x.shape[1]), _ptr(order)))
    return order


class Codebook:
    """DFlash2Codebook: host copy of a [rank, n_rows] selector codebook in ggml storage."""

    def __init__(self, dtype, rank, n_rows, raw):
        raw = np.ascontiguousarray(np.frombuffer(bytes(raw), dtype=np.uint8))
        self.rank, self.n_rows = rank, n_rows
        self.h = C.c_void_p()
        check(lib().dfl_codebook_create(C.c_int32(dtype), C.c_uint64(rank), C.c_uint64(n_rows), _ptr(raw) if raw.size else None,
                                        C.c_uint64(raw.size), C.byref(self.h)))

    def dequant_row(self, row):
        out = np.zeros(self.rank, dtype=np.float32)
        check(lib().dfl_codebook_dequant_row(self.h, C.c_uint64(row), _ptr(out), C.c_uint64(out.size)))
        return out

    def close(self):
        if self.h:
            lib().dfl_codebook_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def selector_walk(predecessor, successor, top_k, rank, carry, n, ids, vals, sel_h):
    """select_draft_path's greedy walk: (tokens[n], scores[n][top_k], scored[n][top_k])."""
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    vals = np.ascontiguousarray(vals, dtype=np.float32)
    sel_h = np.ascontiguousarray(sel_h, dtype=np.float32)
    if ids.size != n * top_k or vals.size != n * top_k or sel_h.size != n * rank:
        raise DflError(2, f"expected ids/vals/gate lengths {n * top_k}/{n * top_k}/{n * rank}, got {ids.size}/{vals.size}/{sel_h.size}")
    tokens = np.zeros(n, dtype=np.int32)
    scores = np.full((n, top_k), -np.inf, dtype=np.float32)
    scored = np.zeros((n, top_k), dtype=np.uint8)
    check(lib().dfl_selector_walk(predecessor.h, successor.h, C.c_uint32(top_k), C.c_uint32(rank), C.c_int32(carry), C.c_uint32(n), _ptr(ids),
                                  _ptr(vals), _ptr(sel_h), _ptr(tokens), _ptr(scores), _ptr(scored)))
    return tokens, scores, scored


def selector_walk_sampled(predecessor, successor, top_k, rank, carry, n, ids, vals, sel_h, proposal_sampler):
    """draft_block_sampled's walk: (tokens[n], [(token, [(cand, weight), ...]) per draft row])."""
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    vals = np.ascontiguousarray(vals, dtype=np.float32)
    sel_h = np.ascontiguousarray(sel_h, dtype=np.float32)
    tokens = np.zeros(n, dtype=np.int32)
    offs = np.zeros(n, dtype=np.uint32)
    ct = np.zeros(max(1, (n - 1) * top_k), dtype=np.int32)
    cw = np.zeros(max(1, (n - 1) * top_k), dtype=np.float64)
    check(lib().dfl_selector_walk_sampled(predecessor.h, successor.h, C.c_uint32(top_k), C.c_uint32(rank), C.c_int32(carry), C.c_uint32(n),
                                          _ptr(ids), _ptr(vals), _ptr(sel_h), proposal_sampler.h, _ptr(tokens), _ptr(offs), _ptr(ct), _ptr(cw)))
    props = [(int(tokens[r + 1]), [(int(ct[k]), float(cw[k])) for k in range(int(offs[r]), int(offs[r + 1]))]) for r in range(n - 1)]
    return tokens, props


def splitmix64_stream(seed, n):
    st = C.c_uint64(seed)
    return [int(lib().dfl_splitmix64_next(C.byref(st))) for _ in range(n)]


def greedy_token(logits):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    tok = C.c_int32(0)
    check(lib().dfl_greedy_token(_ptr(logits), C.c_uint64(logits.size), C.byref(tok)))
    return int(tok.value)


def accept_prefix(verified_tokens, target_logits, vocab, proposals, sampler, remaining_output_budget, stop_ids):
    """proposals: None or list of (token, [(cand_token, weight), ...]).  Returns AcceptDecision as a dict."""
    vt = np.ascontiguousarray(verified_tokens, dtype=np.int32)
    tl = np.ascontiguousarray(target_logits, dtype=np.float32).reshape(-1)
    stops = np.ascontiguousarray(stop_ids, dtype=np.int32)
    sp = None
    keep = []
    if proposals is not None:
        toks = np.ascontiguousarray([p[0] for p in proposals], dtype=np.int32)
        offs = np.zeros(len(proposals) + 1, dtype=np.uint32)
        ct, cw = [], []
        for i, p in enumerate(proposals):
            for t, w in p[1]:
                ct.append(t)
                cw.append(w)
            offs[i + 1] = len(ct)
        ct = np.ascontiguousarray(ct, dtype=np.int32)
        cw = np.ascontiguousarray(cw, dtype=np.float64)
        keep = [toks, offs, ct, cw]
        sp = SparseProposals(len(proposals), _ptr(toks, C.POINTER(C.c_int32)), _ptr(offs, C.POINTER(C.c_uint32)),
                             _ptr(ct, C.POINTER(C.c_int32)), _ptr(cw, C.POINTER(C.c_double)))
    out = AcceptDecision()
    vocab = int(vocab) & ((1 << 64) - 1)
    check(lib().dfl_accept_prefix(_ptr(vt) if vt.size else None, C.c_uint32(vt.size), _ptr(tl) if tl.size else None, C.c_uint64(tl.size),
                                  C.c_uint64(vocab), C.byref(sp) if sp is not None else None, sampler.h,
                                  C.c_uint64(remaining_output_budget), _ptr(stops) if stops.size else None, C.c_uint32(stops.size),
                                  C.byref(out)))
    kinds = {0: None, 1: "correction", 2: "bonus"}
    stopsn = {0: None, 1: "eos", 2: "token_limit"}
    return {"accepted_drafts": list(out.accepted_drafts[:out.n_accepted]),
            "next_carry": (kinds[out.next_carry_kind], out.next_carry) if out.next_carry_kind else None,
            "stop_reason": stopsn[out.stop_reason], "retain_input_count": int(out.retain_input_count), "error_row": out.error_row}


# ---------------------------------------------------------------------------
# drafter / drafter session / outer loop
# ---------------------------------------------------------------------------
class Drafter:
    def __init__(self, target: Model, cfg: DFlashConfig, tensors):
        arr, keep = make_tensor_table(tensors)
        self.target, self.cfg = target, cfg
        self.h = C.c_void_p()
        check(lib().dfl_drafter_create(target.h, C.byref(cfg), arr, C.c_uint64(len(tensors)), C.byref(self.h)))

    @classmethod
    def from_gguf(cls, target, gguf):
        self = cls.__new__(cls)
        self.target, self.cfg = target, gguf.dflash_config(target.arch)
        self.h = C.c_void_p()
        tab, n = gguf.drafter_table()
        check(lib().dfl_drafter_create(target.h, C.byref(self.cfg), tab, C.c_uint64(n), C.byref(self.h)))
        return self

    def weight_bytes(self):
        return int(lib().dfl_drafter_weight_bytes(self.h))

    def layer_ids(self):
        return [int(self.cfg.target_layer_ids[i]) for i in range(self.cfg.n_target_layers)]

    def close(self):
        if self.h:
            lib().dfl_drafter_destroy(self.h)
            self.h = C.c_void_p()


class DSession:
    def __init__(self, drafter: Drafter, ctx_capacity):
        self.drafter = drafter
        self.h = C.c_void_p()
        check(lib().dfl_dsession_create(drafter.h, C.c_uint32(ctx_capacity), C.byref(self.h)))

    @property
    def ctx_len(self):
        return int(lib().dfl_dsession_ctx_len(self.h))

    def append_columns(self, cols, positions):
        cols = np.ascontiguousarray(cols, dtype=np.float32)
        pos = np.ascontiguousarray(positions, dtype=np.uint32)
        check(lib().dfl_dsession_append_columns_host(self.h, _ptr(cols), _ptr(pos), C.c_uint32(pos.size)))

    def append_from_scratch(self, scratch, first_row, count, first_position):
        check(lib().dfl_dsession_append_from_scratch(self.h, scratch.h, C.c_uint32(first_row), C.c_uint32(count), C.c_uint32(first_position)))

    def reset(self):
        check(lib().dfl_dsession_reset(self.h))

    def draft_block_sampled(self, carry, noise_start_pos, proposal_sampler):
        """DFlashDecoder::draft_block_sampled: (tokens[n], [(token, [(cand, weight), ...]) per draft row])."""
        n = self.drafter.cfg.block_size
        out = np.zeros(n, dtype=np.int32)
        offs = np.zeros(n, dtype=np.uint32)
        ct = np.zeros((n - 1) * 16, dtype=np.int32)
        cw = np.zeros((n - 1) * 16, dtype=np.float64)
        check(lib().dfl_draft_block_sampled(self.h, C.c_int32(int(carry)), C.c_uint32(noise_start_pos), proposal_sampler.h, _ptr(out),
                                            _ptr(offs), _ptr(ct), _ptr(cw)))
        props = [(int(out[r + 1]), [(int(ct[k]), float(cw[k])) for k in range(int(offs[r]), int(offs[r + 1]))]) for r in range(n - 1)]
        return out, props

    def read_selector(self):
        """Top-16 ids / logits [n][16] and (with a selector) the gate rows [n][rank] of the last draft pass."""
        n, rank = self.drafter.cfg.block_size, self.drafter.cfg.selector_rank
        ids = np.zeros((n, 16), dtype=np.int32)
        vals = np.zeros((n, 16), dtype=np.float32)
        sel_h = np.zeros((n, rank), dtype=np.float32) if rank else None
        check(lib().dfl_dsession_read_selector(self.h, _ptr(ids), _ptr(vals), _ptr(sel_h) if rank else None))
        return ids, vals, sel_h

    def draft_block(self, carry, noise_start_pos, want_logits=False):
        n = self.drafter.cfg.block_size
        out = np.zeros(n, dtype=np.int32)
        logits = np.zeros((n, self.drafter.target.arch.vocab_size), dtype=np.float32) if want_logits else None
        check(lib().dfl_draft_block(self.h, C.c_int32(int(carry)), C.c_uint32(noise_start_pos), _ptr(out),
                                    _ptr(logits) if want_logits else None))
        return out, logits

    def close(self):
        if self.h:
            lib().dfl_dsession_destroy(self.h)
            self.h = C.c_void_p()


def prefill(model, session, scratch, layer_ids, ids, start_position=0, feed_drafter=None, want_hidden=False, want_logits=True):
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    lids = _u32(layer_ids)
    hidden = np.zeros((ids.size, scratch.k, model.arch.hidden_size), dtype=np.float32) if want_hidden else None
    logits = np.zeros(model.arch.vocab_size, dtype=np.float32) if want_logits else None
    check(lib().dfl_prefill(model.h, session.h, scratch.h, _ptr(lids) if lids.size else None, C.c_uint32(lids.size), _ptr(ids),
                            C.c_uint64(ids.size), C.c_uint32(start_position), feed_drafter.h if feed_drafter is not None else None,
                            _ptr(hidden) if want_hidden else None, _ptr(logits) if want_logits else None))
    return logits, hidden


def generate(model, session, scratch, dsession, sampler, first_logits, max_tokens, stop_ids=(), replay_history=None,
             sparse_proposals=False, verify_margin=0.0, replay_runs_drafter=False, replay_unchecked=False,
             device_row_order=False):
    first_logits = np.ascontiguousarray(first_logits, dtype=np.float32)
    stops = np.ascontiguousarray(stop_ids, dtype=np.int32)
    hist = np.ascontiguousarray(replay_history, dtype=np.int32) if replay_history is not None else None
    p = GenerateParams()
    p.max_tokens = max_tokens
    p.stop_ids = _ptr(stops, C.POINTER(C.c_int32)) if stops.size else None
    p.n_stop_ids = stops.size
    p.replay_history = _ptr(hist, C.POINTER(C.c_int32)) if hist is not None else None
    p.n_replay_history = hist.size if hist is not None else 0
    p.sparse_proposals = 1 if sparse_proposals else 0
    p.verify_margin = verify_margin
    p.replay_runs_drafter = 1 if replay_runs_drafter else 0
    p.replay_unchecked = 1 if replay_unchecked else 0
    p.device_row_order = 1 if device_row_order else 0
    out = np.zeros(max_tokens, dtype=np.int32)
    n = C.c_uint32(0)
    stats = GenerateStats()
    check(lib().dfl_generate(model.h, session.h, scratch.h, dsession.h, sampler.h, _ptr(first_logits), C.byref(p), _ptr(out), C.byref(n),
                             C.byref(stats)))
    return out[:n.value].copy(), stats


class GGUF:
    """A mapped GGUF file: tensor table, typed metadata, the derived Arch / DFlashConfig."""

    def __init__(self, path):
        self.h = C.c_void_p()
        check(lib().dfl_gguf_open(str(path).encode(), C.byref(self.h)))

    def close(self):
        if self.h:
            lib().dfl_gguf_close(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def n_tensors(self):
        return int(lib().dfl_gguf_tensor_count(self.h))

    def table(self):
        """(pointer to the dfl_tensor table, count): pass to Model.from_table / Drafter.from_table."""
        return lib().dfl_gguf_tensors(self.h), self.n_tensors

    def drafter_table(self):
        tab, n = C.POINTER(Tensor)(), C.c_uint64(0)
        check(lib().dfl_gguf_drafter_tensors(self.h, C.byref(tab), C.byref(n)))
        return tab, int(n.value)

    def tensors(self):
        tab, n = self.table()
        return [tab[i] for i in range(n)]

    def find(self, name):
        t = Tensor()
        check(lib().dfl_gguf_find(self.h, name.encode(), C.byref(t)))
        return t

    @staticmethod
    def tensor_bytes(t):
        return np.ctypeslib.as_array(C.cast(t.data, C.POINTER(C.c_uint8)), shape=(int(t.n_bytes),)).copy() if t.n_bytes else np.zeros(0, np.uint8)

    def get_u64(self, key):
        v, f = C.c_uint64(0), C.c_int32(0)
        check(lib().dfl_gguf_get_u64(self.h, key.encode(), C.byref(v), C.byref(f)))
        return int(v.value) if f.value else None

    def get_f64(self, key):
        v, f = C.c_double(0), C.c_int32(0)
        check(lib().dfl_gguf_get_f64(self.h, key.encode(), C.byref(v), C.byref(f)))
        return float(v.value) if f.value else None

    def get_bool(self, key):
        v, f = C.c_int32(0), C.c_int32(0)
        check(lib().dfl_gguf_get_bool(self.h, key.encode(), C.byref(v), C.byref(f)))
        return bool(v.value) if f.value else None

    def get_str(self, key):
        buf, f = C.create_string_buffer(4096), C.c_int32(0)
        check(lib().dfl_gguf_get_str(self.h, key.encode(), buf, C.c_uint64(4096), C.byref(f)))
        return buf.value.decode() if f.value else None

    def get_u64_array(self, key):
        n, f = C.c_uint64(0), C.c_int32(0)
        check(lib().dfl_gguf_get_u64_array(self.h, key.encode(), None, C.c_uint64(0), C.byref(n), C.byref(f)))
        if not f.value:
            return None
        out = np.zeros(max(1, int(n.value)), dtype=np.uint64)
        check(lib().dfl_gguf_get_u64_array(self.h, key.encode(), _ptr(out), C.c_uint64(out.size), C.byref(n), C.byref(f)))
        return [int(x) for x in out[:int(n.value)]]

    def arch(self):
        a = Arch()
        check(lib().dfl_gguf_arch(self.h, C.byref(a)))
        return a

    def dflash_config(self, target_arch):
        c = DFlashConfig()
        check(lib().dfl_gguf_dflash_config(self.h, C.byref(target_arch), C.byref(c)))
        return c


def gemm_timing_begin():
    lib().dfl_gemm_timing_begin()


def gemm_timing_end():
    ms, n, b = C.c_double(0), C.c_uint64(0), C.c_uint64(0)
    check(lib().dfl_gemm_timing_end(C.byref(ms), C.byref(n), C.byref(b)))
    return float(ms.value), int(n.value), int(b.value)


def synth_tensor(name, dtype, n_in, n_out, seed, std, device=0, shape=None):
    """A seeded N(0, std) tensor quantised on the GPU.  Returns (name, dtype, shape, device_ptr, n_bytes)."""
    ptr, nb = C.c_void_p(), C.c_uint64(0)
    check(lib().dfl_synth_tensor(C.c_int32(device), C.c_int32(dtype), C.c_uint64(n_in), C.c_uint64(n_out), C.c_uint64(seed),
                                 C.c_float(std), C.byref(ptr), C.byref(nb)))
    return (name, dtype, shape or [n_in, n_out], ptr.value, int(nb.value))


def device_free(ptr, device=0):
    check(lib().dfl_device_free(C.c_int32(device), C.c_void_p(ptr)))


def device_to_host(ptr, n_bytes, device=0):
    out = np.zeros(n_bytes, dtype=np.uint8)
    check(lib().dfl_device_to_host(C.c_int32(device), C.c_void_p(ptr), _ptr(out), C.c_uint64(n_bytes)))
    return out


def make_device_tensor_table(entries):
    """entries: (name, dtype, shape, ptr_or_ndarray, n_bytes or None); ints are device pointers, arrays host data."""
    arr = (Tensor * len(entries))()
    keep = []
    for i, (name, dtype, shape, data, nb) in enumerate(entries):
        nm = name.encode()
        arr[i].name = nm
        arr[i].dtype = dtype
        arr[i].n_dims = len(shape)
        for j, d in enumerate(shape):
            arr[i].shape[j] = d
        if isinstance(data, int):
            arr[i].data = data
            arr[i].n_bytes = nb
            arr[i].on_device = 1
            keep.append(nm)
        else:
            raw = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
            arr[i].data = raw.ctypes.data
            arr[i].n_bytes = raw.size
            arr[i].on_device = 0
            keep.append((nm, raw))
    return arr, keep
