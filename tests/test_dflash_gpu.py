"""Drafter, prefill and the DFlash outer loop on the GPU against the CPU oracle and against the
reference's end-to-end equivalences (greedy DFlash output == plain greedy decode, PERF-LOG.md:22177-22187;
sampled one-hot coupling keeps the serial RNG stream, sampling.rs:692-703)."""
import numpy as np
import pytest

import modelgen
import orc
from dflb import pkg

pytestmark = pytest.mark.gpu
RTOL, ATOL = 1e-2, 1e-3


@pytest.fixture(scope="module")
def world():
    arch = modelgen.tiny_arch()
    T = modelgen.target_tensors(arch, seed=3)
    cfg = modelgen.tiny_dflash_config(arch)
    D = modelgen.drafter_tensors(arch, cfg, seed=4)
    om, gm = modelgen.OracleModel(arch, T), pkg.Model(arch, T)
    od, gd = modelgen.OracleDrafter(cfg, D), pkg.Drafter(gm, cfg, D)
    yield arch, cfg, om, gm, od, gd
    gd.close(); gm.close()


def test_draft_block_matches_oracle(world):
    arch, cfg, om, gm, od, gd = world
    rng = np.random.default_rng(8)
    layer_ids = gd.layer_ids()
    prompt = rng.integers(0, arch.vocab_size, size=21)
    sess, scr, ds = pkg.Session(gm, 128), pkg.Scratch(gm, 16, len(layer_ids)), pkg.DSession(gd, 128)
    logits, hidden = pkg.prefill(gm, sess, scr, layer_ids, prompt, 0, feed_drafter=ds, want_hidden=True)
    assert ds.ctx_len == 21 and sess.kv_n_pos == 21
    # oracle prefill: hidden captures + last logits
    ost = om.new_state(128, True)
    caps = []
    for i, t in enumerate(prompt):
        l, c = om.single_token(ost, t, i, layer_ids)
        caps.append(c.reshape(-1))
    np.testing.assert_allclose(hidden.reshape(21, -1), np.stack(caps), rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(logits, l, rtol=RTOL, atol=ATOL)
    carry = int(np.argmax(l))
    noise = [carry] + [cfg.mask_token_id] * 15
    # feed the oracle drafter the GPU's own captured context so that only the drafter is compared
    want = od.draft(om, noise, hidden.reshape(21, -1), np.arange(21), 21)
    toks, got = ds.draft_block(carry, 21, want_logits=True)
    np.testing.assert_allclose(got, want, rtol=RTOL, atol=ATOL)
    cos = (got * want).sum(1) / np.sqrt((got * got).sum(1) * (want * want).sum(1))
    assert cos.min() > 0.999            # tests/dflash_correctness.rs:322
    assert toks[0] == carry
    s = np.sort(want, axis=1)
    safe = (s[:, -1] - s[:, -2]) > 1e-4
    want_tok = np.array([orc.greedy_token(r) for r in want])
    assert np.array_equal(toks[1:][safe[1:]], want_tok[1:][safe[1:]])
    # incremental context: a second call after appending more columns equals a fresh session fed everything
    more = rng.integers(0, arch.vocab_size, size=5)
    pkg.packed_verify(gm, sess, scr, layer_ids, more, 21)
    ds.append_from_scratch(scr, 0, 5, 21)
    _, inc = ds.draft_block(carry, 26, want_logits=True)
    ds2 = pkg.DSession(gd, 128)
    ds2.append_columns(hidden.reshape(21, -1), np.arange(21))
    ds2.append_columns(scr.read_capture(5).reshape(5, -1), np.arange(21, 26))
    _, fresh = ds2.draft_block(carry, 26, want_logits=True)
    assert inc.tobytes() == fresh.tobytes()
    # overflow is an error, not a wrap
    with pytest.raises(pkg.DflError) as e:
        ds2.append_columns(np.zeros((128, hidden.shape[1] * hidden.shape[2]), dtype=np.float32), np.arange(128))
    assert e.value.name == "CTX_OVERFLOW"
    for x in (sess, scr, ds, ds2):
        x.close()


def plain_decode(gm, prompt, n_tokens, sampler, layer_ids):
    sess, scr = pkg.Session(gm, 256), pkg.Scratch(gm, 16, len(layer_ids))
    logits, _ = pkg.prefill(gm, sess, scr, layer_ids, prompt, 0)
    out = []
    tok, _ = sampler.sample(logits)
    while True:
        out.append(tok)
        if len(out) == n_tokens:
            break
        logits, _ = pkg.single_token(gm, sess, scr, layer_ids, tok, sess.kv_n_pos, want_hidden=False)
        tok, _ = sampler.sample(logits)
    sess.close(); scr.close()
    return np.array(out, dtype=np.int32)


def dflash_decode(world, prompt, n_tokens, sampler, **kw):
    arch, cfg, om, gm, od, gd = world
    layer_ids = gd.layer_ids()
    sess, scr, ds = pkg.Session(gm, 256), pkg.Scratch(gm, 16, len(layer_ids)), pkg.DSession(gd, 256)
    logits, _ = pkg.prefill(gm, sess, scr, layer_ids, prompt, 0, feed_drafter=ds)
    toks, stats = pkg.generate(gm, sess, scr, ds, sampler, logits, n_tokens, **kw)
    for x in (sess, scr, ds):
        x.close()
    return toks, stats


def test_greedy_dflash_equals_plain_greedy_decode(world):
    arch, cfg, om, gm, od, gd = world
    prompt = np.random.default_rng(9).integers(0, arch.vocab_size, size=19)
    plain = plain_decode(gm, prompt, 40, pkg.Sampler(), gd.layer_ids())
    spec, stats = dflash_decode(world, prompt, 40, pkg.Sampler())
    assert np.array_equal(plain, spec)
    assert stats.verify_calls == stats.spec_steps and stats.tokens_emitted == 40


def test_replayed_drafts_accept_fully_and_partially(world):
    arch, cfg, om, gm, od, gd = world
    prompt = np.random.default_rng(10).integers(0, arch.vocab_size, size=17)
    plain = plain_decode(gm, prompt, 64, pkg.Sampler(), gd.layer_ids())
    # history == the true continuation: every draft is accepted (16 tokens per step)
    spec, stats = dflash_decode(world, prompt, 48, pkg.Sampler(), replay_history=plain)
    assert np.array_equal(spec, plain[:48])
    # the last step stops at the token limit with its terminal token unconsumed, which is one rollback
    assert stats.spec_steps == 3 and stats.accepted_drafts == 45 and stats.restore_calls <= 1 and stats.drafter_calls == 0
    # corrupt one token: the step that meets it accepts a strict prefix and rolls back, output unchanged
    bad = plain.copy()
    bad[20] = (bad[20] + 1) % arch.vocab_size
    spec2, stats2 = dflash_decode(world, prompt, 48, pkg.Sampler(), replay_history=bad)
    assert np.array_equal(spec2, plain[:48])
    assert stats2.restore_calls >= 1


def test_sampled_one_hot_coupling_keeps_the_serial_stream(world):
    arch, cfg, om, gm, od, gd = world
    prompt = np.random.default_rng(12).integers(0, arch.vocab_size, size=23)
    kw = dict(temperature=0.7, top_p=0.95, seed=1234)
    plain = plain_decode(gm, prompt, 36, pkg.Sampler(**kw), gd.layer_ids())
    s = pkg.Sampler(**kw)
    spec, stats = dflash_decode(world, prompt, 36, s)
    assert np.array_equal(plain, spec)
    # sparse proposals: a valid stream of the right length (distribution-preserving, not stream-identical)
    spec3, stats3 = dflash_decode(world, prompt, 36, pkg.Sampler(**kw), sparse_proposals=True)
    assert spec3.size == 36 and spec3.min() >= 0 and spec3.max() < arch.vocab_size


def test_greedy_loop_matches_oracle_loop(world):
    arch, cfg, om, gm, od, gd = world
    prompt = np.random.default_rng(13).integers(0, arch.vocab_size, size=9)
    ost = om.new_state(64, True)
    for i, t in enumerate(prompt):
        l, _ = om.single_token(ost, t, i)
    want, gaps = [], []
    for i in range(12):
        s = np.sort(l)
        gaps.append(s[-1] - s[-2])
        tok = orc.greedy_token(l)
        want.append(tok)
        l, _ = om.single_token(ost, tok, len(prompt) + i)
    got, _ = dflash_decode(world, prompt, 12, pkg.Sampler())
    n_safe = 0
    while n_safe < 12 and gaps[n_safe] > 1e-4:
        n_safe += 1
    assert n_safe >= 6, "seed gives an early near tie; pick another"
    assert list(got[:n_safe]) == want[:n_safe]


def test_draft_block_with_tensor_core_attention_matches_oracle():
    """A drafter with the usual head grouping (4 query heads per KV head, 128-wide) takes the tensor-core span kernel:
    several 64-key chunks of context, a sliding window on the first layer, full attention on the last."""
    arch = modelgen.tiny_arch()
    T = modelgen.target_tensors(arch, seed=3)
    cfg = modelgen.tiny_dflash_config(arch, n_q_heads=4, n_kv_heads=1, swa_window=40)
    D = modelgen.drafter_tensors(arch, cfg, seed=6)
    om, gm = modelgen.OracleModel(arch, T), pkg.Model(arch, T)
    od, gd = modelgen.OracleDrafter(cfg, D), pkg.Drafter(gm, cfg, D)
    rng = np.random.default_rng(9)
    layer_ids = gd.layer_ids()
    n_ctx = 150
    prompt = rng.integers(0, arch.vocab_size, size=n_ctx)
    for cap in (256, 20000):      # one chunk per span, then several chunks per span
        sess, scr, ds = pkg.Session(gm, 256), pkg.Scratch(gm, 16, len(layer_ids)), pkg.DSession(gd, cap)
        logits, hidden = pkg.prefill(gm, sess, scr, layer_ids, prompt, 0, feed_drafter=ds, want_hidden=True)
        hidden = hidden.reshape(n_ctx, -1)
        carry = int(np.argmax(logits))
        noise = [carry] + [cfg.mask_token_id] * 15
        want = od.draft(om, noise, hidden, np.arange(n_ctx), n_ctx)
        toks, got = ds.draft_block(carry, n_ctx, want_logits=True)
        np.testing.assert_allclose(got, want, rtol=RTOL, atol=ATOL)
        cos = (got * want).sum(1) / np.sqrt((got * got).sum(1) * (want * want).sum(1))
        assert cos.min() > 0.999
        # a context with a gap in its positions (columns dropped from the middle) still follows the position mask
        ds2 = pkg.DSession(gd, cap)
        keep = np.r_[0:60, 100:150]
        ds2.append_columns(hidden[keep], keep)
        want2 = od.draft(om, noise, hidden[keep], keep, n_ctx)
        _, got2 = ds2.draft_block(carry, n_ctx, want_logits=True)
        np.testing.assert_allclose(got2, want2, rtol=RTOL, atol=ATOL)
        for x in (sess, scr, ds, ds2):
            x.close()
    gd.close(); gm.close()


@pytest.mark.parametrize("causal", [0, 1])
def test_drafter_attention_over_the_tiled_context_matches_oracle(monkeypatch, causal):
    # the full-attention layer of a long drafter session reads a tiled f16 hi + lo shadow of its f32 context through
    # the tcgen05 kernel: forced on here for a 300-column context (three tiles + the block's own tile, one tile per
    # span), positions with gaps, bidirectional and causal; checked against the oracle and against the row-major path
    arch = modelgen.tiny_arch()
    cfg = modelgen.tiny_dflash_config(arch, n_q_heads=4, causal=causal)
    T, D = modelgen.target_tensors(arch, seed=3), modelgen.drafter_tensors(arch, cfg, seed=6)
    om, gm = modelgen.OracleModel(arch, T), pkg.Model(arch, T)
    od, gd = modelgen.OracleDrafter(cfg, D), pkg.Drafter(gm, cfg, D)
    rng = np.random.default_rng(12)
    n_ctx = 300
    ctx = (rng.standard_normal((n_ctx, cfg.n_target_layers * arch.hidden_size)) * 0.5).astype(np.float32)
    pos = np.cumsum(rng.integers(1, 3, size=n_ctx)).astype(np.uint32)      # increasing, with gaps
    start = int(pos[-1]) + 1 if causal else int(pos[n_ctx // 2])            # bidirectional: later context columns too
    carry = 11
    noise = [carry] + [cfg.mask_token_id] * 15
    want = od.draft(om, noise, ctx, pos, start)
    outs = {}
    for tiled in ("1", "0"):
        monkeypatch.setenv("DFL_DATTN_TILED", tiled)
        ds = pkg.DSession(gd, 384)
        ds.append_columns(ctx[:250], pos[:250])
        ds.draft_block(carry, start)                                       # a pass in between: the shadow grows incrementally
        ds.append_columns(ctx[250:], pos[250:])
        _, got = ds.draft_block(carry, start, want_logits=True)
        np.testing.assert_allclose(got, want, rtol=RTOL, atol=ATOL, err_msg=f"tiled={tiled}")
        outs[tiled] = got
        ds.close()
    np.testing.assert_allclose(outs["1"], outs["0"], rtol=1e-3, atol=2e-4)
    gd.close(); gm.close()
