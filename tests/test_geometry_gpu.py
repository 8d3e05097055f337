"""Parity with the CPU oracle at the widths the benchmark configurations name, on slices of a few layers:

* the dense 9B-class hybrid (hidden 4096, 32 query / 8 KV heads of 128, GDN 32 value / 16 key heads, FFN 12288,
  vocabulary 151 936, fp16 KV cache) - 3 GDN layers + 1 attention layer;
* the 35B-A3B-shaped routed-expert hybrid (hidden 2048, 16 query / 2 KV heads of 256 = GQA group 8, 256 experts
  top-8 + one shared expert, expert FFN 512) - 1 GDN layer + 1 attention layer;
* the drafter at the dense model's width (hidden 4096, 32 / 8 heads of 128, FFN 12288, 5 tap layers; 2 layers).

Each case runs two 16-row blocks, a partial rollback and a third block through the packed verify and compares
logits, captured hidden rows, recurrent state, KV rows and (routed experts) the chosen expert ids with the oracle
fed the accepted tokens one at a time (forward.rs:173-220, :749-824, :834-932, :940-1107).  The weights are made
on the GPU by the library's seeded generator and copied to the host for the oracle, so both sides decode the same
bytes.  The measured logit error and the share of rows whose oracle top-1 / top-2 gap is below 1e-4 are printed
(run with -s) and, when DFL_PARITY_REPORT_DIR names a directory, written to geometry_parity.json there."""
import importlib
import json
import os

import numpy as np
import pytest

import modelgen
import orc
from dflb import pkg

syn = importlib.import_module("qwen-llm_b200.synthetic")
pytestmark = pytest.mark.gpu
RTOL, ATOL = 1e-2, 1e-3  # logits contract
GAP = 1e-4               # rows with a smaller oracle top-1 / top-2 gap are near ties


def _report(name, stats):
    print(name, json.dumps(stats))
    out = os.environ.get("DFL_PARITY_REPORT_DIR", "")
    if out and os.path.isdir(out):
        path = os.path.join(out, "geometry_parity.json")
        allr = json.load(open(path)) if os.path.exists(path) else {}
        allr[name] = stats
        json.dump(allr, open(path, "w"), indent=1)


def _randomised_norms(entries, seed):
    """The generator's norm weights are ones; move them off one so that a misplaced or skipped norm shows."""
    rng = np.random.default_rng(seed)
    out = []
    for (name, dtype, shape, data, nb) in entries:
        if not isinstance(data, int) and name.endswith("norm.weight"):
            data = (1.0 + 0.1 * rng.standard_normal(data.size)).astype(np.float32)
        out.append((name, dtype, shape, data, nb))
    return out


def _host_copy(entries):
    host = []
    for (name, dtype, shape, data, nb) in entries:
        raw = pkg.device_to_host(data, nb) if isinstance(data, int) else np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        host.append((name, dtype, shape, raw))
    return host


def _build_target(arch, seed):
    ents = _randomised_norms(syn.target_entries(arch, seed=seed, device=0), seed + 1)
    host = _host_copy(ents)
    gm = syn.build_model(arch, ents)
    syn.free_entries(ents)
    return modelgen.OracleModel(arch, host), gm


def _oracle_block(om, st, tokens, start, layer_ids, want_route=False):
    import ctypes as C
    logits, caps, routes = [], [], []
    k = om.arch.expert_used_count
    for i, t in enumerate(tokens):
        l, c = om.single_token(st, t, start + i, layer_ids)
        logits.append(l)
        caps.append(c)
        if want_route:   # the expert ids of the last routed layer, in choice order
            r = np.zeros(k, dtype=np.int32)
            assert om.L.orc_last_route(om.h, r.ctypes.data_as(C.c_void_p), C.c_uint32(k)) == k
            routes.append(r)
    return np.stack(logits), np.stack(caps), (np.stack(routes) if want_route else None)


def _check_block(name, om, ost, gm, sess, scr, layer_ids, tokens, start, stats, moe=False):
    want, want_cap, want_route = _oracle_block(om, ost, tokens, start, layer_ids, want_route=moe)
    am, gap, got = pkg.packed_verify(gm, sess, scr, layer_ids, tokens, start, want_logits=True)
    np.testing.assert_allclose(got, want, rtol=RTOL, atol=ATOL, err_msg=name)
    np.testing.assert_allclose(scr.read_capture(len(tokens)), want_cap, rtol=RTOL, atol=ATOL, err_msg=name)
    s = np.sort(want, axis=1)
    og = s[:, -1] - s[:, -2]
    want_arg = np.array([orc.greedy_token(r) for r in want])
    safe = og > GAP
    assert np.array_equal(am[safe], want_arg[safe]), name
    np.testing.assert_allclose(gap, og, rtol=0, atol=2e-3)
    if moe:
        assert np.array_equal(scr.read_route(len(tokens)), want_route), name + ": expert ids"
    denom = np.maximum(np.abs(want), 1e-3)
    stats["max_rel_err"] = max(stats.get("max_rel_err", 0.0), float((np.abs(got - want) / denom).max()))
    stats["max_abs_err"] = max(stats.get("max_abs_err", 0.0), float(np.abs(got - want).max()))
    stats["rows"] = stats.get("rows", 0) + len(tokens)
    stats["near_tie_rows"] = stats.get("near_tie_rows", 0) + int((~safe).sum())
    stats["argmax_equal_rows"] = stats.get("argmax_equal_rows", 0) + int((am == want_arg).sum())
    stats["min_gap"] = min(stats.get("min_gap", 1e9), float(og.min()))


def _verify_rollback_case(name, arch, seed, n_gdn, moe=False, warm_blocks=0):
    om, gm = _build_target(arch, seed)
    rng = np.random.default_rng(seed + 2)
    layer_ids = [0, arch.n_layer - 1]
    cap = 16 * (warm_blocks + 4)
    sess, scr = pkg.Session(gm, cap, True), pkg.Scratch(gm, 16, len(layer_ids))
    ost = om.new_state(cap, True)
    stats = {}
    pos = 0
    for _ in range(warm_blocks):   # context for several 64-position KV chunks
        toks = rng.integers(0, arch.vocab_size, size=16)
        pkg.packed_verify(gm, sess, scr, layer_ids, toks, pos)
        for i, t in enumerate(toks):
            om.single_token(ost, t, pos + i, (), want_logits=False)
        pos += 16
    toks = rng.integers(0, arch.vocab_size, size=16)
    _check_block(name, om, ost, gm, sess, scr, layer_ids, toks, pos, stats, moe)
    pos += 16
    # second block: verified in full, then rolled back to 6 of its rows; the oracle is fed those 6 only
    toks = rng.integers(0, arch.vocab_size, size=16)
    _check_block(name, om, om.clone_state(ost), gm, sess, scr, layer_ids, toks, pos, stats, moe)
    n_keep = 6
    pkg.restore_partial(gm, sess, scr, n_keep, pos)
    for i in range(n_keep):
        om.single_token(ost, toks[i], pos + i, (), want_logits=False)
    pos += n_keep
    assert sess.kv_n_pos == pos
    for gi in range(n_gdn):
        ssm, conv = sess.read_gdn_state(gi)
        wssm, wconv = om.read_gdn(ost, gi)
        np.testing.assert_allclose(ssm, wssm, rtol=RTOL, atol=ATOL, err_msg=f"{name}: recurrent state {gi} after rollback")
        np.testing.assert_allclose(conv, wconv, rtol=RTOL, atol=ATOL, err_msg=f"{name}: conv state {gi} after rollback")
    toks = rng.integers(0, arch.vocab_size, size=16)
    _check_block(name, om, ost, gm, sess, scr, layer_ids, toks, pos, stats, moe)
    pos += 16
    for p in (0, pos - 17, pos - 1):   # KV rows: first, the last kept row of the rolled-back block, the newest
        k, v = sess.read_kv(0, p)
        wk, wv = om.read_kv(ost, 0, p)
        np.testing.assert_allclose(k, wk, rtol=RTOL, atol=ATOL, err_msg=f"{name}: K row {p}")
        np.testing.assert_allclose(v, wv, rtol=RTOL, atol=ATOL, err_msg=f"{name}: V row {p}")
    for gi in range(n_gdn):
        ssm, conv = sess.read_gdn_state(gi)
        wssm, wconv = om.read_gdn(ost, gi)
        np.testing.assert_allclose(ssm, wssm, rtol=RTOL, atol=ATOL)
        np.testing.assert_allclose(conv, wconv, rtol=RTOL, atol=ATOL)
    stats["near_tie_fraction"] = stats["near_tie_rows"] / stats["rows"]
    _report(name, stats)
    sess.close(); scr.close(); gm.close()


def _slice_arch(base, n_layer, interval):
    a = pkg.Arch()
    for f, _ in base._fields_:
        setattr(a, f, getattr(base, f))
    a.n_layer, a.full_attention_interval = n_layer, interval
    return a


def test_dense_9b_widths_verify_and_rollback_match_oracle():
    # 8 KV heads, 32 value / 16 key GDN heads, vocabulary 151 936; five warm-up blocks put the checked blocks past
    # the first 64-position KV chunk
    arch = _slice_arch(syn.arch_9b(), 4, 4)
    _verify_rollback_case("dense_9b_widths", arch, seed=41, n_gdn=3, warm_blocks=5)


def test_dense_9b_widths_with_the_tiled_kv_cache(monkeypatch):
    # the same slice over the tiled fp16 cache (tcgen05 attention kernel): 8 KV heads' tiles side by side, nine warm-up
    # blocks so that the checked blocks attend over two 128-position tiles (two spans at this capacity)
    monkeypatch.setenv("DFL_ATTN_TILED", "1")
    arch = _slice_arch(syn.arch_9b(), 4, 4)
    _verify_rollback_case("dense_9b_widths_tiled_kv", arch, seed=41, n_gdn=3, warm_blocks=9)


def test_routed_35b_a3b_widths_verify_and_rollback_match_oracle():
    # 256-wide heads in a GQA group of 8 over 2 KV heads; 256 experts, top-8, plus the shared expert
    arch = _slice_arch(syn.arch_35b_a3b(), 2, 2)
    _verify_rollback_case("routed_35b_a3b_widths", arch, seed=43, n_gdn=1, moe=True, warm_blocks=5)


def test_drafter_at_dense_9b_widths_matches_oracle():
    arch = _slice_arch(syn.arch_9b(), 4, 4)
    om, gm = _build_target(arch, seed=41)
    cfg = syn.dflash_config_9b(arch)
    cfg.n_layer = 2
    cfg.layer_is_swa[0], cfg.layer_is_swa[1] = 1, 0
    cfg.swa_window = 24     # the context below is longer than the window, so the first layer's mask matters
    for i, l in enumerate([0, 1, 2, 3, 3][:cfg.n_target_layers]):
        cfg.target_layer_ids[i] = l
    dents = _randomised_norms(syn.drafter_entries(arch, cfg, seed=5, device=0), 6)
    od = modelgen.OracleDrafter(cfg, _host_copy(dents))
    gd = syn.build_drafter(gm, cfg, dents)
    syn.free_entries(dents)
    rng = np.random.default_rng(7)
    layer_ids = gd.layer_ids()
    n_prompt = 40
    prompt = rng.integers(0, arch.vocab_size, size=n_prompt)
    sess, scr, ds = pkg.Session(gm, 128), pkg.Scratch(gm, 16, len(layer_ids)), pkg.DSession(gd, 128)
    logits, hidden = pkg.prefill(gm, sess, scr, layer_ids, prompt, 0, feed_drafter=ds, want_hidden=True)
    carry = int(np.argmax(logits))
    noise = [carry] + [cfg.mask_token_id] * 15
    # the oracle drafter is fed the GPU's own captured context, so that only the drafter is compared
    want = od.draft(om, noise, hidden.reshape(n_prompt, -1), np.arange(n_prompt), n_prompt)
    toks, got = ds.draft_block(carry, n_prompt, want_logits=True)
    np.testing.assert_allclose(got, want, rtol=RTOL, atol=ATOL)
    cos = (got * want).sum(1) / np.sqrt((got * got).sum(1) * (want * want).sum(1))
    assert cos.min() > 0.999
    s = np.sort(want, axis=1)
    safe = (s[:, -1] - s[:, -2]) > GAP
    want_tok = np.array([orc.greedy_token(r) for r in want])
    assert np.array_equal(toks[1:][safe[1:]], want_tok[1:][safe[1:]])
    denom = np.maximum(np.abs(want), 1e-3)
    _report("drafter_dense_9b_widths", {"max_rel_err": float((np.abs(got - want) / denom).max()), "max_abs_err": float(np.abs(got - want).max()),
                                        "rows": 16, "near_tie_rows": int((~safe).sum()), "min_cos": float(cos.min())})
    for x in (sess, scr, ds, gd, gm):
        x.close()


@pytest.mark.parametrize("moe", [False, True])
def test_a_repeated_verify_from_the_same_state_gives_the_same_bits(moe):
    """One packed verify repeated from the same session state, at the benchmark widths (every weight format and ring
    depth of the few-row GEMM, the 151 936-row head included): logits and captured rows must not change by a bit.
    This is the check that caught a group of the GEMM taking the other group's outstanding weight copy for its own."""
    arch = _slice_arch(syn.arch_35b_a3b(), 2, 2) if moe else _slice_arch(syn.arch_9b(), 4, 4)
    ents = syn.target_entries(arch, seed=47, device=0)
    gm = syn.build_model(arch, ents)
    syn.free_entries(ents)
    layer_ids = [0, 1] if moe else [0, 1, 2, 3]
    sess, scr = pkg.Session(gm, 256, True), pkg.Scratch(gm, 16, len(layer_ids))
    rng = np.random.default_rng(6)
    pkg.packed_verify(gm, sess, scr, layer_ids, rng.integers(0, arch.vocab_size, size=16), 0)
    pos = sess.kv_n_pos
    toks = rng.integers(0, arch.vocab_size, size=16)
    first = None
    for _ in range(60):
        am, gap, logits = pkg.packed_verify(gm, sess, scr, layer_ids, toks, pos, want_logits=True)
        got = (logits.tobytes(), scr.read_capture(16).tobytes(), am.tobytes())
        if first is None:
            first = got
        assert got == first
        pkg.restore_pre_block(gm, sess, scr, pos)
    sess.close(); scr.close(); gm.close()
