"""Seeded synthetic hybrid target / drafter builders shared by tests, smoke and bench.
Weights ~ N(0, std) quantised with the oracle's block packers in the Q4_K_M dtype mix the
reference reports for production files (attention q/k/v/o Q4_K; FFN gate/up Q4_K, down Q6_K;
GDN in_proj_qkv Q6_K, in_proj_z Q4_K, out_proj Q5_K, alpha/beta f32; lm_head Q6_K; token_embd Q4_K;
norms f32; drafter bf16)."""
import numpy as np

import orc
from dflb import pkg


def tiny_arch(**kw):
    a = pkg.Arch()
    d = dict(n_layer=4, hidden_size=256, intermediate_size=512, vocab_size=1000, full_attention_interval=4, n_q_heads=2,
             n_kv_heads=1, attn_head_dim=128, rope_theta=10000000.0, partial_rotary_factor=0.25, gdn_n_v_heads=2, gdn_n_k_heads=1,
             gdn_head_dim=128, gdn_conv_kernel=4, expert_count=0, expert_used_count=0, expert_feed_forward_length=0,
             expert_shared_feed_forward_length=0)
    d.update(kw)
    for k, v in d.items():
        setattr(a, k, v)
    return a


def is_attn(arch, il):
    iv = max(arch.full_attention_interval, 1)
    return il % iv == iv - 1


def target_tensors(arch, seed=0, std=0.02, embd_dtype=orc.Q4_K, head_dtype=orc.Q6_K, tied=False):
    rng = np.random.default_rng(seed)
    H, F, V = arch.hidden_size, arch.intermediate_size, arch.vocab_size
    hd = arch.attn_head_dim
    q_dim, kv_dim = arch.n_q_heads * hd, arch.n_kv_heads * hd
    n_v, n_k = arch.gdn_n_v_heads, arch.gdn_n_k_heads
    conv_dim, v_dim = (2 * n_k + n_v) * 128, n_v * 128
    T = []

    def mat(name, dtype, n_in, n_out, s=std):
        w = (rng.standard_normal((n_out, n_in)) * s).astype(np.float32)
        T.append((name, dtype, [n_in, n_out], orc.quantize(dtype, w)))

    def vec(name, values):
        T.append((name, orc.F32, [values.size], np.ascontiguousarray(values, dtype=np.float32).view(np.uint8)))

    def norm(name, n):
        vec(name, 1.0 + 0.1 * rng.standard_normal(n))

    mat("token_embd.weight", embd_dtype, H, V, 1.0)
    if not tied:
        mat("output.weight", head_dtype, H, V)
    norm("output_norm.weight", H)
    for il in range(arch.n_layer):
        b = f"blk.{il}."
        norm(b + "attn_norm.weight", H)
        norm(b + "post_attention_norm.weight", H)
        if is_attn(arch, il):
            mat(b + "attn_q.weight", orc.Q4_K, H, 2 * q_dim)
            mat(b + "attn_k.weight", orc.Q4_K, H, kv_dim)
            mat(b + "attn_v.weight", orc.Q4_K, H, kv_dim)
            mat(b + "attn_output.weight", orc.Q4_K, q_dim, H)
            norm(b + "attn_q_norm.weight", hd)
            norm(b + "attn_k_norm.weight", hd)
        else:
            mat(b + "attn_qkv.weight", orc.Q6_K, H, conv_dim)
            mat(b + "attn_gate.weight", orc.Q4_K, H, v_dim)
            mat(b + "ssm_out.weight", orc.Q5_K, v_dim, H)
            T.append((b + "ssm_alpha.weight", orc.F32, [H, n_v], (rng.standard_normal((n_v, H)) * std).astype(np.float32).view(np.uint8)))
            T.append((b + "ssm_beta.weight", orc.F32, [H, n_v], (rng.standard_normal((n_v, H)) * std).astype(np.float32).view(np.uint8)))
            vec(b + "ssm_a", -rng.uniform(0.1, 2.0, n_v))
            vec(b + "ssm_dt.bias", rng.uniform(-1.0, 1.0, n_v))
            T.append((b + "ssm_conv1d.weight", orc.F32, [4, conv_dim], (rng.standard_normal((conv_dim, 4)) * 0.3).astype(np.float32).view(np.uint8)))
            norm(b + "ssm_norm.weight", 128)
        if arch.expert_count > 0:
            # routed experts stacked along the last ggml dimension (expert-major contiguous) + one shared expert
            E, Fe, Fs = arch.expert_count, arch.expert_feed_forward_length, arch.expert_shared_feed_forward_length
            T.append((b + "ffn_gate_inp.weight", orc.F32, [H, E], (rng.standard_normal((E, H)) * 0.5).astype(np.float32).view(np.uint8)))
            for nm in ("ffn_gate_exps.weight", "ffn_up_exps.weight"):
                w = (rng.standard_normal((E * Fe, H)) * std).astype(np.float32)
                T.append((b + nm, orc.Q4_K, [H, Fe, E], orc.quantize(orc.Q4_K, w)))
            w = (rng.standard_normal((E * H, Fe)) * std).astype(np.float32)
            T.append((b + "ffn_down_exps.weight", orc.Q6_K, [Fe, H, E], orc.quantize(orc.Q6_K, w)))
            vec(b + "ffn_gate_inp_shexp.weight", rng.standard_normal(H) * 0.1)
            mat(b + "ffn_gate_shexp.weight", orc.Q4_K, H, Fs)
            mat(b + "ffn_up_shexp.weight", orc.Q4_K, H, Fs)
            mat(b + "ffn_down_shexp.weight", orc.Q6_K, Fs, H)
        else:
            mat(b + "ffn_gate.weight", orc.Q4_K, H, F)
            mat(b + "ffn_up.weight", orc.Q4_K, H, F)
            mat(b + "ffn_down.weight", orc.Q6_K, F, H)
    return T


class OracleModel:
    """Oracle-side model + state with the same tensor table."""

    def __init__(self, arch, tensors):
        import ctypes as C
        self.arch = arch
        arr, self._keep = pkg.make_tensor_table(tensors)
        self.L = orc.lib()
        self.h = C.c_void_p(self.L.orc_model_create(C.byref(arch), arr, C.c_uint64(len(tensors))))
        assert self.h, self.L.orc_last_error()

    def new_state(self, kv_capacity, kv_f16):
        import ctypes as C
        return C.c_void_p(self.L.orc_state_create(self.h, C.c_uint64(kv_capacity), C.c_int32(1 if kv_f16 else 0)))

    def clone_state(self, st):
        import ctypes as C
        return C.c_void_p(self.L.orc_state_clone(st))

    def single_token(self, st, token, position, layer_ids=(), want_logits=True):
        import ctypes as C
        ids = np.ascontiguousarray(layer_ids, dtype=np.uint32)
        cap = np.zeros((max(1, ids.size), self.arch.hidden_size), dtype=np.float32)
        logits = np.zeros(self.arch.vocab_size, dtype=np.float32)
        p = lambda a: a.ctypes.data_as(C.c_void_p)
        orc.check(self.L.orc_single_token(self.h, st, C.c_int32(int(token)), C.c_uint32(position), p(ids), C.c_uint32(ids.size),
                                          p(cap) if ids.size else None, p(logits) if want_logits else None, None))
        return logits, cap

    def read_gdn(self, st, gi):
        import ctypes as C
        a = self.arch
        ssm = np.zeros(a.gdn_n_v_heads * 128 * 128, dtype=np.float32)
        conv = np.zeros(3 * (2 * a.gdn_n_k_heads + a.gdn_n_v_heads) * 128, dtype=np.float32)
        p = lambda x: x.ctypes.data_as(C.c_void_p)
        assert self.L.orc_state_read_gdn(st, C.c_uint32(gi), p(ssm), p(conv)) == 0
        return ssm, conv

    def last_route(self, cap=64):
        """Expert ids the last routed-expert call chose (the model's last MoE layer of the last token)."""
        import ctypes as C
        out = np.zeros(cap, dtype=np.int32)
        n = int(self.L.orc_last_route(self.h, out.ctypes.data_as(C.c_void_p), C.c_uint32(cap)))
        return [int(v) for v in out[:n]]

    def read_kv(self, st, ai, pos):
        import ctypes as C
        n = self.arch.n_kv_heads * self.arch.attn_head_dim
        k = np.zeros(n, dtype=np.float32)
        v = np.zeros(n, dtype=np.float32)
        p = lambda x: x.ctypes.data_as(C.c_void_p)
        assert self.L.orc_state_read_kv(self.h, st, C.c_uint32(ai), C.c_uint32(pos), p(k), p(v)) == 0
        return k, v


def tiny_dflash_config(arch, **kw):
    c = pkg.DFlashConfig()
    d = dict(n_layer=2, hidden_size=arch.hidden_size, intermediate_size=512, n_q_heads=2, n_kv_heads=1, head_dim=128,
             rope_theta=1000000.0, rms_norm_eps=1e-6, causal=0, swa_window=8, block_size=16, mask_token_id=7, n_target_layers=2)
    d.update(kw)
    for k, v in d.items():
        setattr(c, k, v)
    ids = kw.get("ids", [1, arch.n_layer - 1])
    for i, l in enumerate(ids[:c.n_target_layers]):
        c.target_layer_ids[i] = l
    swa = kw.get("swa", [1] * (c.n_layer - 1) + [0])     # sliding window on all but the last layer
    for i, v in enumerate(swa[:c.n_layer]):
        c.layer_is_swa[i] = v
    return c


def drafter_tensors(arch, cfg, seed=1, std=0.02, dtype=orc.BF16, codebook_dtype=orc.Q8_0, selector_std=0.05):
    rng = np.random.default_rng(seed)
    H, F = cfg.hidden_size, cfg.intermediate_size
    q_dim, kv_dim = cfg.n_q_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
    KH = cfg.n_target_layers * arch.hidden_size
    T = []

    def mat(name, n_in, n_out, s=std):
        w = (rng.standard_normal((n_out, n_in)) * s).astype(np.float32)
        T.append((name, dtype, [n_in, n_out], orc.quantize(dtype, w)))

    def norm(name, n):
        T.append((name, orc.F32, [n], (1.0 + 0.1 * rng.standard_normal(n)).astype(np.float32).view(np.uint8)))

    mat("dflash_fc.weight", KH, H)
    norm("dflash_hidden_norm.weight", H)
    norm("output_norm.weight", H)
    for il in range(cfg.n_layer):
        b = f"blk.{il}."
        norm(b + "attn_norm.weight", H)
        norm(b + "post_attention_norm.weight", H)
        norm(b + "attn_q_norm.weight", cfg.head_dim)
        norm(b + "attn_k_norm.weight", cfg.head_dim)
        mat(b + "attn_q.weight", H, q_dim)
        mat(b + "attn_k.weight", H, kv_dim)
        mat(b + "attn_v.weight", H, kv_dim)
        mat(b + "attn_output.weight", q_dim, H)
        mat(b + "ffn_gate.weight", H, F)
        mat(b + "ffn_up.weight", H, F)
        mat(b + "ffn_down.weight", F, H)
    if cfg.selector_rank:   # DFlash 2 selector tensors (loader.rs:1182-1230)
        rank, V = cfg.selector_rank, arch.vocab_size
        mat("selector_hidden.weight", H, rank, s=selector_std)
        for name in ("selector_predecessor.weight", "selector_successor.weight"):
            w = (rng.standard_normal((V, rank)) * 0.5).astype(np.float32)
            T.append((name, codebook_dtype, [rank, V], orc.quantize(codebook_dtype, w)))
    return T


class OracleDrafter:
    def __init__(self, cfg, tensors):
        import ctypes as C
        self.cfg = cfg
        arr, self._keep = pkg.make_tensor_table(tensors)
        self.L = orc.lib()
        self.h = C.c_void_p(self.L.orc_drafter_create(C.byref(cfg), arr, C.c_uint64(len(tensors))))
        assert self.h, self.L.orc_last_error()

    def draft(self, target: "OracleModel", noise_ids, ctx_stacked, pos_ctx, noise_start):
        import ctypes as C
        noise = np.ascontiguousarray(noise_ids, dtype=np.int32)
        ctx = np.ascontiguousarray(ctx_stacked, dtype=np.float32)
        pos = np.ascontiguousarray(pos_ctx, dtype=np.uint32)
        out = np.zeros((noise.size, target.arch.vocab_size), dtype=np.float32)
        p = lambda a: a.ctypes.data_as(C.c_void_p)
        orc.check(self.L.orc_dflash_draft(self.h, target.h, p(noise), C.c_uint32(noise.size), p(ctx), C.c_uint32(pos.size), p(pos),
                                          C.c_uint32(noise_start), p(out)))
        return out

    def draft_hidden(self, target: "OracleModel", noise_ids, ctx_stacked, pos_ctx, noise_start):
        """logits [n][V] and the rows after output_norm [n][H]"""
        import ctypes as C
        noise = np.ascontiguousarray(noise_ids, dtype=np.int32)
        ctx = np.ascontiguousarray(ctx_stacked, dtype=np.float32)
        pos = np.ascontiguousarray(pos_ctx, dtype=np.uint32)
        out = np.zeros((noise.size, target.arch.vocab_size), dtype=np.float32)
        hid = np.zeros((noise.size, self.cfg.hidden_size), dtype=np.float32)
        p = lambda a: a.ctypes.data_as(C.c_void_p)
        orc.check(self.L.orc_dflash_draft_hidden(self.h, target.h, p(noise), C.c_uint32(noise.size), p(ctx), C.c_uint32(pos.size), p(pos),
                                                 C.c_uint32(noise_start), p(out), p(hid)))
        return out, hid
