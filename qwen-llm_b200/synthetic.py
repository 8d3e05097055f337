"""Seeded synthetic hybrid targets and DFlash drafters built on the GPU (no model files needed).

Large matrices are drawn from N(0, std) and quantised on the device by dfl_synth_tensor in the
Q4_K_M dtype mix the reference reports for production files (attention q/k/v/o Q4_K; FFN gate/up
Q4_K, down Q6_K; GDN in_proj_qkv Q6_K, in_proj_z Q4_K, out_proj Q5_K, alpha/beta f32; lm_head Q6_K;
token_embd Q4_K; norms f32 = 1; drafter bf16).  Small vectors come from numpy with the same seed.
"""
import importlib

import numpy as np

pkg = importlib.import_module(__name__.rsplit(".", 1)[0])

F32, F16, Q8_0, Q4_K, Q5_K, Q6_K, BF16 = pkg.F32, pkg.F16, pkg.Q8_0, pkg.Q4_K, pkg.Q5_K, pkg.Q6_K, pkg.BF16


def arch_9b():
    """The dense benchmark target: 9B-class qwen35-style hybrid (32 layers, GDN:attention 3:1, hidden 4096, vocabulary 151 936)."""
    a = pkg.Arch()
    for k, v in dict(n_layer=32, hidden_size=4096, intermediate_size=12288, vocab_size=151936, full_attention_interval=4,
                     n_q_heads=32, n_kv_heads=8, attn_head_dim=128, rope_theta=10000000.0, partial_rotary_factor=0.25,
                     gdn_n_v_heads=32, gdn_n_k_heads=16, gdn_head_dim=128, gdn_conv_kernel=4, expert_count=0, expert_used_count=0,
                     expert_feed_forward_length=0, expert_shared_feed_forward_length=0).items():
        setattr(a, k, v)
    return a


def arch_35b_a3b():
    """The routed-expert benchmark target: 35B-A3B-shaped qwen35moe hybrid (256 routed experts top-8 + one shared expert)."""
    a = pkg.Arch()
    for k, v in dict(n_layer=40, hidden_size=2048, intermediate_size=0, vocab_size=151936, full_attention_interval=4,
                     n_q_heads=16, n_kv_heads=2, attn_head_dim=256, rope_theta=10000000.0, partial_rotary_factor=0.25,
                     gdn_n_v_heads=32, gdn_n_k_heads=16, gdn_head_dim=128, gdn_conv_kernel=4, expert_count=256, expert_used_count=8,
                     expert_feed_forward_length=512, expert_shared_feed_forward_length=512).items():
        setattr(a, k, v)
    return a


def dflash_config_9b(arch):
    """5-layer DFlash-1 shaped drafter: block 16, K=5 evenly spaced tap layers, SWA 2048 on all but the last layer."""
    c = pkg.DFlashConfig()
    k = 5
    for key, v in dict(n_layer=5, hidden_size=arch.hidden_size, intermediate_size=arch.intermediate_size, n_q_heads=32, n_kv_heads=8,
                       head_dim=128, rope_theta=10000000.0, rms_norm_eps=1e-6, causal=0, swa_window=2048, block_size=16,
                       mask_token_id=arch.vocab_size - 1, n_target_layers=k).items():
        setattr(c, key, v)
    for i in range(k):
        c.target_layer_ids[i] = int(round((i + 1) * arch.n_layer / k)) - 1
    for i in range(c.n_layer):
        c.layer_is_swa[i] = 1 if i < c.n_layer - 1 else 0
    return c


def is_attn(arch, il):
    iv = max(arch.full_attention_interval, 1)
    return il % iv == iv - 1


def target_entries(arch, seed=0, std=0.02, device=0, layers=None):
    """Tensor entries for make_device_tensor_table; `layers` restricts to some block indices (plus the globals)."""
    H, F, V = arch.hidden_size, arch.intermediate_size, arch.vocab_size
    hd = arch.attn_head_dim
    q_dim, kv_dim = arch.n_q_heads * hd, arch.n_kv_heads * hd
    n_v, n_k = arch.gdn_n_v_heads, arch.gdn_n_k_heads
    conv_dim, v_dim = (2 * n_k + n_v) * 128, n_v * 128
    rng = np.random.default_rng(seed)
    E = []
    counter = [seed * 1000003 + 17]

    def mat(name, dtype, n_in, n_out, s=std, shape=None):
        counter[0] += 1
        E.append(pkg.synth_tensor(name, dtype, n_in, n_out, counter[0], s, device, shape))

    def vec(name, values, shape=None):
        a = np.ascontiguousarray(values, dtype=np.float32)
        E.append((name, F32, shape or [a.size], a, None))

    mat("token_embd.weight", Q4_K, H, V, 1.0)
    mat("output.weight", Q6_K, H, V)
    vec("output_norm.weight", np.ones(H))
    for il in (range(arch.n_layer) if layers is None else layers):
        b = f"blk.{il}."
        vec(b + "attn_norm.weight", np.ones(H))
        vec(b + "post_attention_norm.weight", np.ones(H))
        if is_attn(arch, il):
            mat(b + "attn_q.weight", Q4_K, H, 2 * q_dim)
            mat(b + "attn_k.weight", Q4_K, H, kv_dim)
            mat(b + "attn_v.weight", Q4_K, H, kv_dim)
            mat(b + "attn_output.weight", Q4_K, q_dim, H)
            vec(b + "attn_q_norm.weight", np.ones(hd))
            vec(b + "attn_k_norm.weight", np.ones(hd))
        else:
            mat(b + "attn_qkv.weight", Q6_K, H, conv_dim)
            mat(b + "attn_gate.weight", Q4_K, H, v_dim)
            mat(b + "ssm_out.weight", Q5_K, v_dim, H)
            mat(b + "ssm_alpha.weight", F32, H, n_v)
            mat(b + "ssm_beta.weight", F32, H, n_v)
            vec(b + "ssm_a", -rng.uniform(0.1, 2.0, n_v))
            vec(b + "ssm_dt.bias", rng.uniform(-1.0, 1.0, n_v))
            vec(b + "ssm_conv1d.weight", rng.standard_normal((conv_dim, 4)) * 0.3, [4, conv_dim])
            vec(b + "ssm_norm.weight", np.ones(128))
        if arch.expert_count > 0:
            # experts stacked along the last ggml dimension: expert gate/up Q4_K, down Q6_K, router f32 (the quantisation mix the reference reports for production files)
            ne, fe, fs = arch.expert_count, arch.expert_feed_forward_length, arch.expert_shared_feed_forward_length
            mat(b + "ffn_gate_inp.weight", F32, H, ne, 0.5)
            mat(b + "ffn_gate_exps.weight", Q4_K, H, ne * fe, shape=[H, fe, ne])
            mat(b + "ffn_up_exps.weight", Q4_K, H, ne * fe, shape=[H, fe, ne])
            mat(b + "ffn_down_exps.weight", Q6_K, fe, ne * H, shape=[fe, H, ne])
            vec(b + "ffn_gate_inp_shexp.weight", rng.standard_normal(H) * 0.1)
            mat(b + "ffn_gate_shexp.weight", Q4_K, H, fs)
            mat(b + "ffn_up_shexp.weight", Q4_K, H, fs)
            mat(b + "ffn_down_shexp.weight", Q6_K, fs, H)
        else:
            mat(b + "ffn_gate.weight", Q4_K, H, F)
            mat(b + "ffn_up.weight", Q4_K, H, F)
            mat(b + "ffn_down.weight", Q6_K, F, H)
    return E


def drafter_entries(arch, cfg, seed=1, std=0.02, device=0, dtype=BF16):
    H, F = cfg.hidden_size, cfg.intermediate_size
    q_dim, kv_dim = cfg.n_q_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
    KH = cfg.n_target_layers * arch.hidden_size
    E = []
    counter = [seed * 7919 + 5]

    def mat(name, n_in, n_out):
        counter[0] += 1
        E.append(pkg.synth_tensor(name, dtype, n_in, n_out, counter[0], std, device))

    def ones(name, n):
        E.append((name, F32, [n], np.ones(n, dtype=np.float32), None))

    mat("dflash_fc.weight", KH, H)
    ones("dflash_hidden_norm.weight", H)
    ones("output_norm.weight", H)
    for il in range(cfg.n_layer):
        b = f"blk.{il}."
        for nm, n in (("attn_norm.weight", H), ("post_attention_norm.weight", H), ("attn_q_norm.weight", cfg.head_dim),
                      ("attn_k_norm.weight", cfg.head_dim)):
            ones(b + nm, n)
        mat(b + "attn_q.weight", H, q_dim)
        mat(b + "attn_k.weight", H, kv_dim)
        mat(b + "attn_v.weight", H, kv_dim)
        mat(b + "attn_output.weight", q_dim, H)
        mat(b + "ffn_gate.weight", H, F)
        mat(b + "ffn_up.weight", H, F)
        mat(b + "ffn_down.weight", F, H)
    return E


def free_entries(entries, device=0):
    for e in entries:
        if isinstance(e[3], int):
            pkg.device_free(e[3], device)


class _Handle:
    pass


def build_model(arch, entries, device=0, ep=None):
    """ep = (rank, world, nccl_id): the expert-parallel slice of a routed-expert model (see pkg.Model)."""
    import ctypes as C
    arr, keep = pkg.make_device_tensor_table(entries)
    m = pkg.Model.__new__(pkg.Model)
    m.arch, m.device = arch, device
    m.h = C.c_void_p()
    if ep is None:
        pkg.check(pkg.lib().dfl_model_create(C.c_int32(device), C.byref(arch), arr, C.c_uint64(len(entries)), C.byref(m.h)))
    else:
        rank, world, nccl_id = ep
        idb = (C.c_uint8 * 128).from_buffer_copy(nccl_id)
        pkg.check(pkg.lib().dfl_model_create_ep(C.c_int32(device), C.byref(arch), arr, C.c_uint64(len(entries)), C.c_int32(rank),
                                                C.c_int32(world), idb, C.byref(m.h)))
    return m


def build_drafter(target, cfg, entries):
    import ctypes as C
    arr, keep = pkg.make_device_tensor_table(entries)
    d = pkg.Drafter.__new__(pkg.Drafter)
    d.target, d.cfg = target, cfg
    d.h = C.c_void_p()
    pkg.check(pkg.lib().dfl_drafter_create(target.h, C.byref(cfg), arr, C.c_uint64(len(entries)), C.byref(d.h)))
    return d
