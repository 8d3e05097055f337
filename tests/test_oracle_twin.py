"""Cross-implementation agreement of the oracle: the C++ restatement of the reference's CPU forward (oracle/forward.hpp,
its own block decoders) against the numpy restatement (oracle/forward_np.py, the gguf package's decoders), token by
token on small dense and routed-expert hybrids.  The two were written separately against forward.rs; they differ only in
summation order, so they must agree far inside the GPU contract (rtol 1e-2 / atol 1e-3)."""
import importlib.util
import os

import numpy as np
import pytest

import modelgen

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
spec = importlib.util.spec_from_file_location("forward_np", os.path.join(ROOT, "oracle", "forward_np.py"))
fnp = importlib.util.module_from_spec(spec)
spec.loader.exec_module(fnp)


def _run_both(arch, seed, n_tokens, kv_f16, moe=False):
    T = modelgen.target_tensors(arch, seed=seed)
    om = modelgen.OracleModel(arch, T)
    nm = fnp.Model(arch, T)
    ost, nst = om.new_state(64, kv_f16), nm.new_state(kv_f16)
    rng = np.random.default_rng(seed + 1)
    ids = [0, arch.n_layer - 1]
    worst = 0.0
    for pos in range(n_tokens):
        tok = int(rng.integers(0, arch.vocab_size))
        a, ca = om.single_token(ost, tok, pos, ids)
        b, cb = nm.single_token(nst, tok, pos, ids)
        np.testing.assert_allclose(b, a, rtol=1e-3, atol=1e-4, err_msg=f"logits at position {pos}")
        np.testing.assert_allclose(cb, ca, rtol=1e-3, atol=1e-4, err_msg=f"captured hidden rows at position {pos}")
        assert int(np.argmax(a)) == int(np.argmax(b)) or np.sort(a)[-1] - np.sort(a)[-2] < 1e-4
        if moe:
            assert sorted(om.last_route()[:arch.expert_used_count]) == sorted(nst.last_route)
        worst = max(worst, float(np.abs(a - b).max()))
    # state after the run: the recurrent state and the conv window of the first GDN layer, a KV row
    ssm, conv = om.read_gdn(ost, 0)
    np.testing.assert_allclose(nst.ssm[0].reshape(-1), ssm, rtol=1e-3, atol=1e-5)
    np.testing.assert_allclose(nst.conv[0].reshape(-1), conv, rtol=1e-3, atol=1e-5)
    k, v = om.read_kv(ost, 0, n_tokens - 1)
    il = nm.attn_layers[0]
    np.testing.assert_allclose(nst.k[il][-1].reshape(-1), k, rtol=1e-3, atol=1e-5)
    np.testing.assert_allclose(nst.v[il][-1].reshape(-1), v, rtol=1e-3, atol=1e-5)
    return worst


@pytest.mark.parametrize("kv_f16", [False, True])
def test_dense_hybrid_agrees(kv_f16):
    worst = _run_both(modelgen.tiny_arch(n_q_heads=4), seed=5, n_tokens=6, kv_f16=kv_f16)
    assert worst < 1e-3


def test_routed_expert_hybrid_agrees():
    arch = modelgen.tiny_arch(expert_count=8, expert_used_count=2, expert_feed_forward_length=256, expert_shared_feed_forward_length=256)
    worst = _run_both(arch, seed=9, n_tokens=5, kv_f16=False, moe=True)
    assert worst < 1e-3


def test_primitives_agree_with_the_reference_known_answers():
    # forward.rs:1377-1414 on the numpy side as well
    x = np.array([1.0, 2.0, 3.0, 4.0], dtype=np.float32)
    y = fnp.rms_norm(x, np.ones(4, dtype=np.float32), np.float32(0.0))
    assert abs(float(np.mean(y * y)) - 1.0) < 1e-5
    assert abs(float(fnp.silu(np.float32(0.0)))) < 1e-7
    assert abs(float(fnp.sigmoid(np.float32(0.0))) - 0.5) < 1e-7
    assert abs(float(fnp.softplus(np.float32(30.0))) - 30.0) < 1e-6
    assert abs(float(fnp.softplus(np.float32(-30.0))) - float(np.exp(np.float32(-30.0)))) < 1e-12
    p = fnp.softmax(np.array([1.0, 2.0, 3.0], dtype=np.float32))
    assert abs(float(p.sum()) - 1.0) < 1e-6 and p[2] > p[1] > p[0]


@pytest.mark.parametrize("swa,causal", [(8, 0), (0, 0), (6, 1)])
def test_drafter_agrees(swa, causal):
    # forward.rs:380-662: context columns at arbitrary positions, sliding-window and full layers, bidirectional or causal
    arch = modelgen.tiny_arch()
    cfg = modelgen.tiny_dflash_config(arch, swa_window=swa, causal=causal)
    T, D = modelgen.target_tensors(arch, seed=3), modelgen.drafter_tensors(arch, cfg, seed=4)
    om, od = modelgen.OracleModel(arch, T), modelgen.OracleDrafter(cfg, D)
    nm, nd = fnp.Model(arch, T), fnp.Drafter(cfg, D)
    rng = np.random.default_rng(11)
    n_ctx = 13
    ctx = (rng.standard_normal((n_ctx, cfg.n_target_layers * arch.hidden_size)) * 0.5).astype(np.float32)
    pos_ctx = np.arange(n_ctx, dtype=np.uint32) + 2
    noise = rng.integers(0, arch.vocab_size, size=16)
    want, want_h = od.draft_hidden(om, noise, ctx, pos_ctx, 15)
    got, got_h = nd.draft(nm, noise, ctx, pos_ctx, 15)
    np.testing.assert_allclose(got_h, want_h, rtol=1e-3, atol=1e-4)
    np.testing.assert_allclose(got, want, rtol=1e-3, atol=1e-4)
