"""Packed verify / single token / rollback of the hybrid target against the CPU oracle
(the reference's model-witness tests, crates/qwen-llm/src/metal_dflash/tests.rs:5887-7700, restated on a
seeded synthetic model)."""
import numpy as np
import pytest

import modelgen
import orc
from dflb import pkg

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-2, 1e-3  # logits contract


@pytest.fixture(scope="module")
def tiny():
    arch = modelgen.tiny_arch()
    T = modelgen.target_tensors(arch, seed=3)
    om = modelgen.OracleModel(arch, T)
    gm = pkg.Model(arch, T)
    yield arch, om, gm
    gm.close()


def oracle_block(om, st, tokens, start, layer_ids):
    logits, caps = [], []
    for i, t in enumerate(tokens):
        l, c = om.single_token(st, t, start + i, layer_ids)
        logits.append(l)
        caps.append(c)
    return np.stack(logits), np.stack(caps)


@pytest.mark.parametrize("kv_f16", [False, True])
def test_packed_verify_matches_oracle(tiny, kv_f16):
    arch, om, gm = tiny
    rng = np.random.default_rng(1)
    layer_ids = [0, 2, 3]
    sess = pkg.Session(gm, 64, kv_f16)
    scr = pkg.Scratch(gm, 16, len(layer_ids))
    ost = om.new_state(64, kv_f16)
    start = 0
    for n in (16, 5, 16, 1):
        tokens = rng.integers(0, arch.vocab_size, size=n)
        want_logits, want_cap = oracle_block(om, ost, tokens, start, layer_ids)
        am, gap, logits = pkg.packed_verify(gm, sess, scr, layer_ids, tokens, start, want_logits=True)
        np.testing.assert_allclose(logits, want_logits, rtol=RTOL, atol=ATOL)
        cap = scr.read_capture(n)
        np.testing.assert_allclose(cap, want_cap, rtol=RTOL, atol=ATOL)
        want_arg = np.array([orc.greedy_token(r) for r in want_logits])
        s = np.sort(want_logits, axis=1)
        safe = (s[:, -1] - s[:, -2]) > 1e-4       # rows whose argmax is not a near tie in the oracle
        assert np.array_equal(am[safe], want_arg[safe])
        np.testing.assert_allclose(gap, s[:, -1] - s[:, -2], rtol=0, atol=2e-3)
        start += n
        assert sess.kv_n_pos == start
    # state parity
    for gi in range(3):
        ssm, conv = sess.read_gdn_state(gi)
        wssm, wconv = om.read_gdn(ost, gi)
        np.testing.assert_allclose(ssm, wssm, rtol=RTOL, atol=ATOL)
        np.testing.assert_allclose(conv, wconv, rtol=RTOL, atol=ATOL)
    k, v = sess.read_kv(0, start - 1)
    wk, wv = om.read_kv(ost, 0, start - 1)
    np.testing.assert_allclose(k, wk, rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(v, wv, rtol=RTOL, atol=ATOL)
    sess.close(); scr.close()


def test_packed_verify_equals_single_token_steps_bitwise(tiny):
    # tests.rs:5887+: packed verify argmax == N single tokens, bitwise state
    arch, om, gm = tiny
    rng = np.random.default_rng(2)
    tokens = rng.integers(0, arch.vocab_size, size=16)
    a, sa = pkg.Session(gm, 64), pkg.Scratch(gm, 16, 1)
    b, sb = pkg.Session(gm, 64), pkg.Scratch(gm, 16, 1)
    _, _, packed = pkg.packed_verify(gm, a, sa, [3], tokens, 0, want_logits=True)
    for i, t in enumerate(tokens):
        logits, _ = pkg.single_token(gm, b, sb, [3], t, i)
        assert logits.tobytes() == packed[i].tobytes(), f"row {i}"
    for gi in range(3):
        s1, c1 = a.read_gdn_state(gi)
        s2, c2 = b.read_gdn_state(gi)
        assert s1.tobytes() == s2.tobytes() and c1.tobytes() == c2.tobytes()
    for x in (a, sa, b, sb):
        x.close()


@pytest.mark.parametrize("n_keep", [1, 8, 15, 16])
def test_restore_then_marker_equals_sequential(tiny, n_keep):
    # tests.rs:6949-7110: restore(n_keep) then one marker token == n_keep sequential tokens then marker
    arch, om, gm = tiny
    rng = np.random.default_rng(5)
    warm = rng.integers(0, arch.vocab_size, size=7)
    tokens = rng.integers(0, arch.vocab_size, size=16)
    marker = 17
    a, sa = pkg.Session(gm, 64), pkg.Scratch(gm, 16, 0)
    b, sb = pkg.Session(gm, 64), pkg.Scratch(gm, 16, 0)
    pkg.packed_verify(gm, a, sa, [], warm, 0)
    pkg.packed_verify(gm, b, sb, [], warm, 0)
    pkg.packed_verify(gm, a, sa, [], tokens, 7)
    pkg.restore_partial(gm, a, sa, n_keep, 7)
    assert a.kv_n_pos == 7 + n_keep
    pkg.packed_verify(gm, b, sb, [], tokens[:n_keep], 7)
    la, _ = pkg.single_token(gm, a, sa, [], marker, 7 + n_keep)
    lb, _ = pkg.single_token(gm, b, sb, [], marker, 7 + n_keep)
    assert la.tobytes() == lb.tobytes()
    for gi in range(3):
        s1, c1 = a.read_gdn_state(gi)
        s2, c2 = b.read_gdn_state(gi)
        assert s1.tobytes() == s2.tobytes() and c1.tobytes() == c2.tobytes()
    for x in (a, sa, b, sb):
        x.close()


def test_restore_pre_block_and_guard_walls(tiny):
    arch, om, gm = tiny
    rng = np.random.default_rng(6)
    tokens = rng.integers(0, arch.vocab_size, size=16)
    a, sa = pkg.Session(gm, 32), pkg.Scratch(gm, 16, 0)
    s0, c0 = a.read_gdn_state(0)
    _, _, l1 = pkg.packed_verify(gm, a, sa, [], tokens, 0, want_logits=True)
    pkg.restore_pre_block(gm, a, sa, 0)
    assert a.kv_n_pos == 0
    s1, c1 = a.read_gdn_state(0)
    assert s0.tobytes() == s1.tobytes() and c0.tobytes() == c1.tobytes()
    _, _, l2 = pkg.packed_verify(gm, a, sa, [], tokens, 0, want_logits=True)
    assert l1.tobytes() == l2.tobytes()
    # guard wall: start must equal kv_n_pos, capacity, token range, n_keep range
    for bad_start in (0, 17):
        with pytest.raises(pkg.DflError) as e:
            pkg.packed_verify(gm, a, sa, [], tokens, bad_start)
        assert e.value.name == "KV_STATE"
    with pytest.raises(pkg.DflError) as e:
        pkg.packed_verify(gm, a, sa, [], np.r_[tokens, [1]], 16)
    assert e.value.name == "BAD_SHAPE"
    bad = tokens.copy()
    bad[3] = arch.vocab_size
    with pytest.raises(pkg.DflError) as e:
        pkg.packed_verify(gm, a, sa, [], bad, 16)
    assert e.value.name == "BAD_TOKEN"
    pkg.packed_verify(gm, a, sa, [], tokens, 16)         # 16 + 16 == capacity: fits
    with pytest.raises(pkg.DflError) as e:
        pkg.packed_verify(gm, a, sa, [], tokens[:1], 32)  # one past capacity
    assert e.value.name == "KV_STATE"
    for bad_keep in (0, 17):
        with pytest.raises(pkg.DflError) as e:
            pkg.restore_partial(gm, a, sa, bad_keep, 16)
        assert e.value.name == "BAD_SHAPE"
    assert not a.poisoned and a.kv_n_pos == 32
    a.close(); sa.close()


def test_injected_completion_failure_poisons_session(tiny):
    # metal/completion.rs:41-66 + metal_forward/mod.rs:2161-2170
    arch, om, gm = tiny
    a, sa = pkg.Session(gm, 32), pkg.Scratch(gm, 16, 0)
    a.fail_next_completion()
    with pytest.raises(pkg.DflError):
        pkg.packed_verify(gm, a, sa, [], [1, 2, 3], 0)
    assert a.poisoned
    with pytest.raises(pkg.DflError) as e:
        pkg.packed_verify(gm, a, sa, [], [1, 2, 3], 3)
    assert e.value.name == "POISONED"
    a.close(); sa.close()


def test_routed_expert_ffn_matches_oracle():
    # forward.rs:749-824 (softmax over all experts, top-k by probability then index, renormalised weights, shared
    # expert behind a sigmoid gate) on a small MoE hybrid; also the packed rows against single-token steps, bitwise
    arch = modelgen.tiny_arch(expert_count=8, expert_used_count=2, expert_feed_forward_length=256,
                              expert_shared_feed_forward_length=256)
    T = modelgen.target_tensors(arch, seed=11)
    om = modelgen.OracleModel(arch, T)
    gm = pkg.Model(arch, T)
    rng = np.random.default_rng(5)
    sess, scr = pkg.Session(gm, 64, False), pkg.Scratch(gm, 16, 1)
    ost = om.new_state(64, False)
    start = 0
    for n in (16, 3):
        tokens = rng.integers(0, arch.vocab_size, size=n)
        want_logits, _ = oracle_block(om, ost, tokens, start, [arch.n_layer - 1])
        am, gap, logits = pkg.packed_verify(gm, sess, scr, [arch.n_layer - 1], tokens, start, want_logits=True)
        np.testing.assert_allclose(logits, want_logits, rtol=RTOL, atol=ATOL)
        start += n
    # packed == sequential single-token steps, bitwise
    sess2, scr2 = pkg.Session(gm, 64, False), pkg.Scratch(gm, 16, 1)
    tokens = rng.integers(0, arch.vocab_size, size=6)
    _, _, packed = pkg.packed_verify(gm, sess2, scr2, [0], tokens, 0, want_logits=True)
    sess3 = pkg.Session(gm, 64, False)
    for i, t in enumerate(tokens):
        row, _ = pkg.single_token(gm, sess3, scr2, [0], int(t), i)
        assert row.tobytes() == packed[i].tobytes()
    for o in (sess, sess2, sess3, scr, scr2):
        o.close()
    gm.close()


@pytest.mark.parametrize("kv_f16", [False, True])
def test_verify_over_a_multi_chunk_kv_cache_with_rollback(tiny, kv_f16):
    # long-context shape of the step in miniature: the block attends over several 64-position KV chunks (partial
    # softmax per chunk + combine), a partial accept rolls KV and GDN state back, and the next block still matches
    # the oracle fed with the accepted tokens only
    arch, om, gm = tiny
    rng = np.random.default_rng(9)
    cap = 384
    sess, scr = pkg.Session(gm, cap, kv_f16), pkg.Scratch(gm, 16, 1)
    ost = om.new_state(cap, kv_f16)
    pos = 0
    while pos < 304:                                  # fill 4.75 chunks through the packed path
        toks = rng.integers(0, arch.vocab_size, size=16)
        pkg.packed_verify(gm, sess, scr, [3], toks, pos)
        for i, t in enumerate(toks):
            om.single_token(ost, t, pos + i, (), want_logits=False)
        pos += 16
    toks = rng.integers(0, arch.vocab_size, size=16)
    want, _ = oracle_block(om, om.clone_state(ost), toks, pos, [3])
    _, _, got = pkg.packed_verify(gm, sess, scr, [3], toks, pos, want_logits=True)
    np.testing.assert_allclose(got, want, rtol=RTOL, atol=ATOL)
    n_keep = 5
    pkg.restore_partial(gm, sess, scr, n_keep, pos)
    for i in range(n_keep):
        om.single_token(ost, toks[i], pos + i, (), want_logits=False)
    pos += n_keep
    toks = rng.integers(0, arch.vocab_size, size=16)
    want, _ = oracle_block(om, ost, toks, pos, [3])
    _, _, got = pkg.packed_verify(gm, sess, scr, [3], toks, pos, want_logits=True)
    np.testing.assert_allclose(got, want, rtol=RTOL, atol=ATOL)
    sess.close(); scr.close()


def test_attention_row_grouping_does_not_change_a_bit(tiny, monkeypatch):
    # long contexts put all 16 rows of a block in one attention CTA per KV chunk, short ones four: same bits
    arch, om, gm = tiny
    rng = np.random.default_rng(13)
    blocks = [rng.integers(0, arch.vocab_size, size=16) for _ in range(6)]
    outs = []
    for rows in ("4", "16"):
        monkeypatch.setenv("DFL_ATTN_ROWS_PER_CTA", rows)
        sess, scr = pkg.Session(gm, 128, True), pkg.Scratch(gm, 16, 1)
        got = []
        for i, b in enumerate(blocks):
            _, _, lg = pkg.packed_verify(gm, sess, scr, [3], b, 16 * i, want_logits=True)
            got.append(lg)
        outs.append(np.concatenate(got))
        sess.close(); scr.close()
    assert outs[0].tobytes() == outs[1].tobytes()


@pytest.fixture(scope="module")
def tiny_g4():
    # GQA group of four 128-wide heads over an fp16 cache: the geometry of the tensor-core attention kernel
    arch = modelgen.tiny_arch(n_q_heads=4)
    T = modelgen.target_tensors(arch, seed=21)
    om = modelgen.OracleModel(arch, T)
    gm = pkg.Model(arch, T)
    yield arch, om, gm
    gm.close()


@pytest.mark.parametrize("cap,tiled", [(384, "0"), (40000, "0"), (384, "1"), (40000, None)])
def test_tensor_core_attention_matches_oracle_and_single_token_steps(tiny_g4, cap, tiled, monkeypatch):
    # row-major cache (mma.sync kernel): cap 384 = one 64-position chunk per record, cap 40000 = several chunks per span
    # (online softmax inside the CTA).  Tiled cache (tcgen05 kernel): forced on at cap 384 (one 128-position tile per
    # span, so the 240 positions make two spans), chosen by the capacity itself at 40000 (two tiles in one span)
    if tiled is None:
        monkeypatch.delenv("DFL_ATTN_TILED", raising=False)
    else:
        monkeypatch.setenv("DFL_ATTN_TILED", tiled)
    arch, om, gm = tiny_g4
    rng = np.random.default_rng(31)
    sess, scr = pkg.Session(gm, cap, True), pkg.Scratch(gm, 16, 1)
    single, scr1 = pkg.Session(gm, cap, True), pkg.Scratch(gm, 16, 1)
    ost = om.new_state(cap, True)
    pos = 0
    for blk_i in range(14):                          # 224 positions = 3.5 chunks
        toks = rng.integers(0, arch.vocab_size, size=16)
        check = blk_i in (0, 5, 13)
        _, _, got = pkg.packed_verify(gm, sess, scr, [3], toks, pos, want_logits=check)
        if check:
            want, _ = oracle_block(om, om.clone_state(ost), toks, pos, [3])
            np.testing.assert_allclose(got, want, rtol=RTOL, atol=ATOL)
        for i, t in enumerate(toks):
            om.single_token(ost, t, pos + i, (), want_logits=False)
            row, _ = pkg.single_token(gm, single, scr1, [3], int(t), pos + i)
            if check:
                assert row.tobytes() == got[i].tobytes(), f"block {blk_i} row {i}"
        pos += 16
    # partial accept, then the next block still matches the oracle
    toks = rng.integers(0, arch.vocab_size, size=16)
    pkg.packed_verify(gm, sess, scr, [3], toks, pos)
    pkg.restore_partial(gm, sess, scr, 7, pos)
    for i in range(7):
        om.single_token(ost, toks[i], pos + i, (), want_logits=False)
    pos += 7
    toks = rng.integers(0, arch.vocab_size, size=16)
    want, _ = oracle_block(om, ost, toks, pos, [3])
    _, _, got = pkg.packed_verify(gm, sess, scr, [3], toks, pos, want_logits=True)
    np.testing.assert_allclose(got, want, rtol=RTOL, atol=ATOL)
    for o in (sess, scr, single, scr1):
        o.close()


@pytest.mark.parametrize("rescale", ["0", "1.5", "12"])
def test_tcgen05_attention_agrees_with_the_oracle_at_any_rescale_threshold(monkeypatch, rescale):
    # the kernel rescales its output accumulator only when a lane's maximum grows by more than a threshold; with the
    # threshold at 0 every new maximum takes the rescale path (classic online softmax), at 12 almost none does.  Wide
    # score ranges (query norm weights x 6) over 2.5 tiles in one span and over three spans.
    monkeypatch.setenv("DFL_ATTN_TILED", "1")
    monkeypatch.setenv("DFL_ATTN_T5_RESCALE", rescale)
    arch = modelgen.tiny_arch(n_q_heads=4)
    T = modelgen.target_tensors(arch, seed=23)
    T = [(n, d, s, (np.frombuffer(bytes(b), dtype=np.float32) * 6.0).astype(np.float32).view(np.uint8)) if n.endswith("attn_q_norm.weight") else (n, d, s, b)
         for n, d, s, b in T]
    om, gm = modelgen.OracleModel(arch, T), pkg.Model(arch, T)
    rng = np.random.default_rng(41)
    for cap in (384, 40000):                         # one tile per span / all tiles in one span
        sess, scr = pkg.Session(gm, cap, True), pkg.Scratch(gm, 16, 1)
        ost = om.new_state(cap, True)
        pos = 0
        for blk_i in range(20):                      # 320 positions
            toks = rng.integers(0, arch.vocab_size, size=16)
            check = blk_i in (0, 8, 15, 19)
            _, _, got = pkg.packed_verify(gm, sess, scr, [3], toks, pos, want_logits=check)
            if check:
                want, _ = oracle_block(om, om.clone_state(ost), toks, pos, [3])
                np.testing.assert_allclose(got, want, rtol=RTOL, atol=ATOL)
            for i, t in enumerate(toks):
                om.single_token(ost, t, pos + i, (), want_logits=False)
            pos += 16
        sess.close(); scr.close()
    gm.close()


def test_tcgen05_attention_block_across_a_tile_boundary_and_at_full_capacity(tiny_g4, monkeypatch):
    # a 16-row block whose rows sit on both sides of a 128-position tile boundary (its first rows see one tile, its last
    # rows two: the new tile holds eight written keys), and a cache filled to its last position
    monkeypatch.setenv("DFL_ATTN_TILED", "1")
    arch, om, gm = tiny_g4
    rng = np.random.default_rng(57)
    cap = 256
    sess, scr = pkg.Session(gm, cap, True), pkg.Scratch(gm, 16, 1)
    ost = om.new_state(cap, True)
    pos = 0
    for n in [16] * 7 + [8]:                          # 120 positions
        toks = rng.integers(0, arch.vocab_size, size=n)
        pkg.packed_verify(gm, sess, scr, [3], toks, pos)
        for i, t in enumerate(toks):
            om.single_token(ost, t, pos + i, (), want_logits=False)
        pos += n
    while pos < cap:                                  # 120-135 straddles the boundary; the last block ends at capacity
        toks = rng.integers(0, arch.vocab_size, size=min(16, cap - pos))
        want, _ = oracle_block(om, ost, toks, pos, [3])
        _, _, got = pkg.packed_verify(gm, sess, scr, [3], toks, pos, want_logits=True)
        np.testing.assert_allclose(got, want, rtol=RTOL, atol=ATOL, err_msg=f"block at {pos}")
        pos += len(toks)
    assert sess.kv_n_pos == cap
    with pytest.raises(pkg.DflError) as e:            # the guard wall still holds
        pkg.packed_verify(gm, sess, scr, [3], [1], pos)
    assert e.value.name == "KV_STATE"
    sess.close(); scr.close()


def test_snapshot_moves_between_tiled_and_row_major_caches(tiny_g4, monkeypatch):
    # a snapshot carries K / V as position-major rows whatever the session's storage: tiled -> tiled continues bitwise,
    # tiled -> rows and rows -> tiled hold the same f16 rows
    arch, om, gm = tiny_g4
    rng = np.random.default_rng(77)
    cap = 384
    monkeypatch.setenv("DFL_ATTN_TILED", "1")
    src, scr = pkg.Session(gm, cap, True), pkg.Scratch(gm, 16, 1)
    pos = 0
    for _ in range(9):                                # 144 positions: one full tile and a partial one
        pkg.packed_verify(gm, src, scr, [3], rng.integers(0, arch.vocab_size, size=16), pos)
        pos += 16
    blob = pkg.session_snapshot(gm, src, None)
    same = pkg.Session(gm, cap, True)
    pkg.session_restore_snapshot(gm, same, None, blob)
    monkeypatch.setenv("DFL_ATTN_TILED", "0")
    rows = pkg.Session(gm, cap, True)
    pkg.session_restore_snapshot(gm, rows, None, blob)
    blob_rows = pkg.session_snapshot(gm, rows, None)
    assert bytes(blob_rows) == bytes(blob)            # rows -> snapshot is the identical byte string
    for p in (0, 127, 128, pos - 1):
        k0, v0 = src.read_kv(0, p)
        for other in (same, rows):
            k1, v1 = other.read_kv(0, p)
            assert k0.tobytes() == k1.tobytes() and v0.tobytes() == v1.tobytes(), p
    toks = rng.integers(0, arch.vocab_size, size=16)
    scr2 = pkg.Scratch(gm, 16, 1)
    _, _, a = pkg.packed_verify(gm, src, scr, [3], toks, pos, want_logits=True)
    _, _, b = pkg.packed_verify(gm, same, scr2, [3], toks, pos, want_logits=True)
    assert a.tobytes() == b.tobytes()
    _, _, c = pkg.packed_verify(gm, rows, scr2, [3], toks, pos, want_logits=True)   # other kernel, same values to tolerance
    np.testing.assert_allclose(c, a, rtol=RTOL, atol=ATOL)
    for o in (src, same, rows, scr, scr2):
        o.close()


def test_repeated_passes_are_bitwise_reproducible():
    """The pass forks work onto side streams (GDN z / alpha-beta projections) and overlaps launches; twenty fresh sessions
    fed the same two blocks must give the same bits every time (a missing dependency shows up as a rare mismatch)."""
    arch = modelgen.tiny_arch()
    gm = pkg.Model(arch, modelgen.target_tensors(arch, seed=3))
    rng = np.random.default_rng(17)
    blocks = [rng.integers(0, arch.vocab_size, size=16), rng.integers(0, arch.vocab_size, size=9)]
    ref = None
    for it in range(20):
        sess, scr = pkg.Session(gm, 64), pkg.Scratch(gm, 16, 2)
        out = []
        pos = 0
        for b in blocks:
            am, gap, logits = pkg.packed_verify(gm, sess, scr, [1, arch.n_layer - 1], b, pos, want_logits=True)
            out.append(logits.tobytes() + scr.read_capture(len(b)).tobytes())
            pos += len(b)
        out.append(b"".join(np.concatenate(sess.read_gdn_state(g)).tobytes() for g in range(2)))
        if ref is None:
            ref = out
        assert out == ref, f"iteration {it} differs"
        sess.close(); scr.close()
    gm.close()


def test_capture_of_a_layer_listed_twice_fills_both_slots(tiny):
    # a drafter whose tap layers repeat (short targets) reads every slot: both must hold the layer's rows of THIS block
    arch, om, gm = tiny
    rng = np.random.default_rng(23)
    one, sone = pkg.Session(gm, 64), pkg.Scratch(gm, 16, 1)
    two, stwo = pkg.Session(gm, 64), pkg.Scratch(gm, 16, 3)
    pos = 0
    for n in (16, 9):    # two different blocks: a slot that is skipped would keep the first block's rows
        toks = rng.integers(0, arch.vocab_size, size=n)
        pkg.packed_verify(gm, one, sone, [2], toks, pos)
        pkg.packed_verify(gm, two, stwo, [2, 2, 1], toks, pos)
        want = sone.read_capture(n)[:, 0]
        got = stwo.read_capture(n)
        assert got[:, 0].tobytes() == want.tobytes() and got[:, 1].tobytes() == want.tobytes()
        assert got[:, 2].tobytes() != want.tobytes()
        pos += n
    for x in (one, sone, two, stwo):
        x.close()


def test_n_eff_override_forms_of_verify_and_restore(tiny):
    # metal_dflash.rs:9055-9094, :15655-15682: None = the scratch's block size; otherwise tokens.len() == n_eff, and
    # the restore is given the same n_eff as the verify it undoes
    arch, om, gm = tiny
    rng = np.random.default_rng(29)
    toks = rng.integers(0, arch.vocab_size, size=16)
    a, sa = pkg.Session(gm, 64), pkg.Scratch(gm, 16, 0)
    b, sb = pkg.Session(gm, 64), pkg.Scratch(gm, 16, 0)
    am_a, _ = pkg.packed_verify_n_eff(gm, a, sa, [], toks, 0, None)
    am_b, _, _ = pkg.packed_verify(gm, b, sb, [], toks, 0)
    assert np.array_equal(am_a, am_b)
    with pytest.raises(pkg.DflError) as e:
        pkg.packed_verify_n_eff(gm, a, sa, [], toks[:9], 16, None)       # None means 16 tokens
    assert e.value.name == "BAD_SHAPE" and "n_eff" in str(e.value)
    for bad in (0, 17):
        with pytest.raises(pkg.DflError) as e:
            pkg.packed_verify_n_eff(gm, a, sa, [], toks[:9], 16, bad)
        assert e.value.name == "BAD_SHAPE" and "n_block=16" in str(e.value)
    am_a, _ = pkg.packed_verify_n_eff(gm, a, sa, [], toks[:9], 16, 9)
    am_b, _, _ = pkg.packed_verify(gm, b, sb, [], toks[:9], 16)
    assert np.array_equal(am_a, am_b)
    with pytest.raises(pkg.DflError):
        pkg.restore_partial_n_eff(gm, a, sa, 4, 16, None)                # the verify ran with n_eff = 9
    with pytest.raises(pkg.DflError):
        pkg.restore_partial_n_eff(gm, a, sa, 10, 16, 9)                  # n_keep beyond n_eff
    pkg.restore_partial_n_eff(gm, a, sa, 4, 16, 9)
    pkg.restore_partial(gm, b, sb, 4, 16)
    assert a.kv_n_pos == b.kv_n_pos == 20
    for gi in range(3):
        assert np.concatenate(a.read_gdn_state(gi)).tobytes() == np.concatenate(b.read_gdn_state(gi)).tobytes()
    for x in (a, sa, b, sb):
        x.close()


def test_a_bounded_device_wait_that_runs_out_poisons_the_session(tiny):
    # the give-up path of the device-side waits: the kernel records why and returns, the completion check maps the
    # error word to TIMEOUT, the session is poisoned, the word is cleared and other sessions are unaffected
    arch, om, gm = tiny
    a, sa = pkg.Session(gm, 32), pkg.Scratch(gm, 16, 0)
    pkg.packed_verify(gm, a, sa, [], [1, 2, 3], 0)
    with pytest.raises(pkg.DflError) as e:
        a.probe_wait_timeout(polls=200)
    assert e.value.name == "TIMEOUT"
    assert a.poisoned
    with pytest.raises(pkg.DflError) as e:
        pkg.packed_verify(gm, a, sa, [], [4], 3)
    assert e.value.name == "POISONED"
    b = pkg.Session(gm, 32)
    am, _, _ = pkg.packed_verify(gm, b, sa, [], [1, 2, 3], 0)             # the next session works; same scratch
    assert am.shape == (3,) and not b.poisoned
    for x in (a, b, sa):
        x.close()


def test_a_non_finite_router_logit_raises_the_route_status_and_poisons():
    # kernels/moe.metal:355-360 (route status NONFINITE) + metal_forward/mod.rs:2161-2170 (poisoning): an Inf in the
    # router weights reaches the routing kernel as a non-finite logit
    arch = modelgen.tiny_arch(expert_count=8, expert_used_count=2, expert_feed_forward_length=256,
                              expert_shared_feed_forward_length=256)
    T = modelgen.target_tensors(arch, seed=11)
    good = pkg.Model(arch, T)
    bad_T = []
    for (name, dtype, shape, raw) in T:
        if name == "blk.1.ffn_gate_inp.weight":
            w = raw.view(np.float32).copy()
            w[5] = np.inf
            raw = w.view(np.uint8)
        bad_T.append((name, dtype, shape, raw))
    bad = pkg.Model(arch, bad_T)
    toks = np.arange(1, 9)
    s1, c1 = pkg.Session(bad, 32), pkg.Scratch(bad, 16, 0)
    with pytest.raises(pkg.DflError) as e:
        pkg.packed_verify(bad, s1, c1, [], toks, 0)
    assert e.value.name == "ROUTE_STATUS" and s1.poisoned
    s2, c2 = pkg.Session(good, 32), pkg.Scratch(good, 16, 0)
    am, _, _ = pkg.packed_verify(good, s2, c2, [], toks, 0)
    assert not s2.poisoned and (am >= 0).all()
    for x in (s1, c1, s2, c2, good, bad):
        x.close()
