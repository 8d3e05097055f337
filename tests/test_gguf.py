"""The product's GGUF reader against files written by the installed `gguf` package: tensor table, typed metadata,
the derived target architecture and drafter configuration (reference behaviour: crates/qwen-llm/src/gguf.rs,
loader.rs:860-1060, :1331-1656), and the header validation.  No GPU needed."""
import os
import struct

import numpy as np
import pytest

import ggufgen
import modelgen
import orc
from dflb import pkg


def sample_tensors():
    rng = np.random.default_rng(3)
    w = (rng.standard_normal((128, 256)) * 0.1).astype(np.float32)
    return [("token_embd.weight", orc.Q4_K, [256, 128], orc.quantize(orc.Q4_K, w)),
            ("output.weight", orc.Q6_K, [256, 128], orc.quantize(orc.Q6_K, w)),
            ("blk.0.attn_q.weight", orc.Q8_0, [256, 128], orc.quantize(orc.Q8_0, w)),
            ("blk.0.ffn_down.weight", orc.Q5_K, [256, 128], orc.quantize(orc.Q5_K, w)),
            ("blk.0.attn_norm.weight", orc.F32, [256], rng.standard_normal(256).astype(np.float32).view(np.uint8)),
            ("blk.0.ssm_conv1d.weight", orc.F32, [4, 96], rng.standard_normal((96, 4)).astype(np.float32).view(np.uint8)),
            ("dflash_fc.weight", orc.BF16, [256, 128], orc.quantize(orc.BF16, w))]


def test_tensor_table_and_metadata_round_trip(tmp_path):
    path = tmp_path / "a.gguf"
    T = sample_tensors()
    meta = {"x.count": 7, "x.big": 1 << 40, "x.scale": 0.25, "x.flag": True, "x.off": False, "x.name": "hello", "x.ids": [3, 1, 4, 1, 5],
            "x.pattern": [True, False, True], "x.words": ["a", "bc"]}
    ggufgen.write_gguf(path, "qwen35", meta, T)
    g = pkg.GGUF(path)
    assert g.n_tensors == len(T)
    got = {t.name.decode(): t for t in g.tensors()}
    for name, dtype, shape, raw in T:
        t = got[name]
        assert t.dtype == dtype and t.n_dims == len(shape) and [int(t.shape[i]) for i in range(t.n_dims)] == shape
        raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
        assert int(t.n_bytes) == raw.size and np.array_equal(pkg.GGUF.tensor_bytes(t), raw)
        f = g.find(name)
        assert f.data == t.data and f.n_bytes == t.n_bytes
    with pytest.raises(pkg.DflError) as e:
        g.find("nope.weight")
    assert e.value.name == "MISSING_TENSOR"
    assert g.get_str("general.architecture") == "qwen35"
    assert g.get_u64("x.count") == 7 and g.get_u64("x.big") == 1 << 40 and g.get_u64("x.absent") is None
    assert g.get_u64("x.name") is None                       # wrong type reads as absent, like GgufFile::get_u64
    assert g.get_f64("x.scale") == 0.25 and g.get_f64("x.count") == 7.0
    assert g.get_bool("x.flag") is True and g.get_bool("x.off") is False and g.get_bool("x.absent") is None
    with pytest.raises(pkg.DflError):
        g.get_bool("x.count")                                # present with another type is an error (gguf.rs:535-544)
    assert g.get_u64_array("x.ids") == [3, 1, 4, 1, 5] and g.get_u64_array("x.pattern") == [1, 0, 1] and g.get_u64_array("x.absent") is None
    with pytest.raises(pkg.DflError):
        g.get_u64_array("x.words")
    g.close()


def test_custom_alignment_is_honoured(tmp_path):
    path = tmp_path / "b.gguf"
    T = sample_tensors()
    ggufgen.write_gguf(path, "qwen35", {}, T, alignment=256)
    g = pkg.GGUF(path)
    assert g.get_u64("general.alignment") == 256
    for (name, dtype, shape, raw), t in zip(T, g.tensors()):
        assert np.array_equal(pkg.GGUF.tensor_bytes(t), np.ascontiguousarray(raw).view(np.uint8).reshape(-1))
    g.close()


def test_arch_from_metadata(tmp_path):
    arch = modelgen.tiny_arch()
    T = modelgen.target_tensors(arch, seed=3)
    meta = ggufgen.arch_meta(arch)
    path = tmp_path / "t.gguf"
    ggufgen.write_gguf(path, "qwen35", meta, T)
    g = pkg.GGUF(path)
    a = g.arch()
    for f, _ in pkg.Arch._fields_:
        want = getattr(arch, f)
        assert getattr(a, f) == pytest.approx(want), f
    g.close()
    # trailing next-token-prediction layers are not part of the main forward; default interval 4; default rope base
    meta2 = dict(meta)
    meta2["qwen35.block_count"] = arch.n_layer + 1
    meta2["qwen35.nextn_predict_layers"] = 1
    del meta2["qwen35.full_attention_interval"], meta2["qwen35.rope.freq_base"]
    ggufgen.write_gguf(path, "qwen35", meta2, T)
    g = pkg.GGUF(path)
    a = g.arch()
    assert a.n_layer == arch.n_layer and a.full_attention_interval == 4 and a.rope_theta == 10000000.0 and a.partial_rotary_factor == 0.25
    g.close()
    for bad in ({"qwen35.attention.head_count_kv": 3}, {"qwen35.embedding_length": 0}, {"qwen35.ssm.conv_kernel": 0}):
        ggufgen.write_gguf(path, "qwen35", {**meta, **bad}, T)
        g = pkg.GGUF(path)
        with pytest.raises(pkg.DflError):
            g.arch()
        g.close()
    ggufgen.write_gguf(path, "llama", meta, T)
    g = pkg.GGUF(path)
    with pytest.raises(pkg.DflError) as e:
        g.arch()
    assert e.value.name == "UNSUPPORTED"
    g.close()


@pytest.mark.parametrize("v2", [False, True])
def test_dflash_config_from_both_key_sets(tmp_path, v2):
    arch = modelgen.tiny_arch()
    cfg = modelgen.tiny_dflash_config(arch, selector_rank=256 if v2 else 0, selector_top_k=16 if v2 else 0)
    D = modelgen.drafter_tensors(arch, cfg, seed=4)
    path = tmp_path / "d.gguf"
    ggufgen.write_gguf(path, "dflash" if v2 else "dflash-draft", ggufgen.drafter_meta(cfg, v2), ggufgen.v2_names(D) if v2 else D)
    g = pkg.GGUF(path)
    c = g.dflash_config(arch)
    for f, _ in pkg.DFlashConfig._fields_:
        a, b = getattr(c, f), getattr(cfg, f)
        if hasattr(a, "__len__"):
            assert list(a) == list(b), f
        else:
            assert a == pytest.approx(b), f
    tab, n = g.drafter_table()
    names = sorted(tab[i].name.decode() for i in range(n))
    assert names == sorted(t[0] for t in D)       # the "dflash" names come back as the names the drafter is created with
    g.close()
    # a mask token outside the target vocabulary, a pattern of the wrong length and (v2) a layer-input id of 0 are refused
    bads = [{("tokenizer.ggml.mask_token_id" if v2 else "dflash-draft.dflash.mask_token_id"): arch.vocab_size},
            {("dflash." if v2 else "dflash-draft.") + "attention.sliding_window_pattern": [True]}]
    if v2:
        bads.append({"dflash.target_layers": [0, 2]})
    for bad in bads:
        ggufgen.write_gguf(path, "dflash" if v2 else "dflash-draft", {**ggufgen.drafter_meta(cfg, v2), **bad}, D)
        g = pkg.GGUF(path)
        with pytest.raises(pkg.DflError):
            g.dflash_config(arch)
        g.close()


def test_header_validation(tmp_path):
    path = tmp_path / "c.gguf"
    ggufgen.write_gguf(path, "qwen35", {"x.count": 1}, sample_tensors())
    blob = open(path, "rb").read()

    def opened(data):
        p = tmp_path / "m.gguf"
        open(p, "wb").write(data)
        return pkg.GGUF(p)

    opened(blob).close()
    with pytest.raises(pkg.DflError):
        opened(b"GGML" + blob[4:])                                   # magic
    with pytest.raises(pkg.DflError):
        opened(blob[:4] + struct.pack("<I", 1) + blob[8:])           # version 1
    with pytest.raises(pkg.DflError):
        opened(blob[:8] + struct.pack("<Q", 10 ** 7) + blob[16:])    # tensor count over the cap
    with pytest.raises(pkg.DflError):
        opened(blob[:len(blob) - 4096])                              # last tensor extends beyond the file
    with pytest.raises(pkg.DflError):
        opened(blob[:64])                                            # truncated inside the metadata
    with pytest.raises(pkg.DflError):
        pkg.GGUF(tmp_path / "absent.gguf")
    p = tmp_path / "s.gguf"
    ggufgen.write_gguf(p, "qwen35", {"split.count": 2}, sample_tensors())
    with pytest.raises(pkg.DflError) as e:
        pkg.GGUF(p)
    assert e.value.name == "UNSUPPORTED"
