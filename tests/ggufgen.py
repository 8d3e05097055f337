"""Writes GGUF files for the tests with the installed `gguf` package (the reader under test is the product's own)."""
import numpy as np
import gguf

import orc

BLOCK = {orc.Q8_0: (32, 34), orc.Q4_K: (256, 144), orc.Q5_K: (256, 176), orc.Q6_K: (256, 210)}


def write_gguf(path, arch_name, meta, tensors, alignment=None):
    """meta: {key: value} (int -> u32, float -> f32, bool, str, list -> array); tensors: (name, dtype, shape ne0-first, raw bytes)."""
    w = gguf.GGUFWriter(str(path), arch_name)
    if alignment:
        w.add_custom_alignment(alignment)
    for k, v in meta.items():
        if isinstance(v, bool):
            w.add_bool(k, v)
        elif isinstance(v, int):
            (w.add_uint64 if v > 0xFFFFFFFF else w.add_uint32)(k, v)
        elif isinstance(v, float):
            w.add_float32(k, v)
        elif isinstance(v, str):
            w.add_string(k, v)
        else:
            w.add_array(k, list(v))
    for name, dtype, shape, raw in tensors:
        raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
        np_shape = list(reversed(shape))
        if dtype == orc.F32:
            w.add_tensor(name, raw.view(np.float32).reshape(np_shape))
        elif dtype == orc.F16:
            w.add_tensor(name, raw.view(np.float16).reshape(np_shape))
        elif dtype == orc.BF16:
            w.add_tensor(name, raw.reshape(np_shape[:-1] + [np_shape[-1] * 2]), raw_dtype=gguf.GGMLQuantizationType.BF16)
        else:
            el, nb = BLOCK[dtype]
            w.add_tensor(name, raw.reshape(np_shape[:-1] + [np_shape[-1] // el * nb]), raw_dtype=gguf.GGMLQuantizationType(dtype))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()


def arch_meta(arch, name="qwen35"):
    p = name + "."
    m = {p + "block_count": arch.n_layer, p + "embedding_length": arch.hidden_size, p + "feed_forward_length": arch.intermediate_size,
         p + "attention.head_count": arch.n_q_heads, p + "attention.head_count_kv": arch.n_kv_heads,
         p + "attention.key_length": arch.attn_head_dim, p + "full_attention_interval": arch.full_attention_interval,
         p + "ssm.state_size": arch.gdn_head_dim, p + "ssm.time_step_rank": arch.gdn_n_v_heads, p + "ssm.group_count": arch.gdn_n_k_heads,
         p + "ssm.conv_kernel": arch.gdn_conv_kernel, p + "rope.freq_base": float(arch.rope_theta)}
    if arch.expert_count:
        m.update({p + "expert_count": arch.expert_count, p + "expert_used_count": arch.expert_used_count,
                  p + "expert_feed_forward_length": arch.expert_feed_forward_length,
                  p + "expert_shared_feed_forward_length": arch.expert_shared_feed_forward_length})
    return m


def drafter_meta(cfg, v2=False):
    p = "dflash." if v2 else "dflash-draft."
    ids = [int(cfg.target_layer_ids[i]) + (1 if v2 else 0) for i in range(cfg.n_target_layers)]
    m = {p + "block_count": cfg.n_layer, p + "embedding_length": cfg.hidden_size, p + "feed_forward_length": cfg.intermediate_size,
         p + "attention.head_count": cfg.n_q_heads, p + "attention.head_count_kv": cfg.n_kv_heads, p + "attention.key_length": cfg.head_dim,
         p + "rope.freq_base": float(cfg.rope_theta), p + "attention.layer_norm_rms_epsilon": float(cfg.rms_norm_eps),
         p + "attention.causal": bool(cfg.causal), p + "attention.sliding_window": cfg.swa_window,
         p + "attention.sliding_window_pattern": [bool(cfg.layer_is_swa[i]) for i in range(cfg.n_layer)]}
    if v2:
        m.update({"dflash.block_size": cfg.block_size, "tokenizer.ggml.mask_token_id": cfg.mask_token_id, "dflash.target_layers": ids})
        if cfg.selector_rank:
            m.update({"dflash.selector_rank": cfg.selector_rank, "dflash.selector_top_k": cfg.selector_top_k})
    else:
        m.update({p + "dflash.block_size": cfg.block_size, p + "dflash.mask_token_id": cfg.mask_token_id, p + "dflash.target_layer_ids": ids,
                  p + "dflash.n_target_features": cfg.n_target_layers * cfg.hidden_size})
    return m


def v2_names(tensors):
    """the "dflash" format's tensor names for a table written with the "dflash-draft" names"""
    out = []
    for name, dtype, shape, raw in tensors:
        if name == "dflash_fc.weight":
            name = "fc.weight"
        elif name == "dflash_hidden_norm.weight":
            name = "enc.output_norm.weight"
        elif name.endswith(".post_attention_norm.weight"):
            name = name.replace(".post_attention_norm.weight", ".ffn_norm.weight")
        out.append((name, dtype, shape, raw))
    return out
