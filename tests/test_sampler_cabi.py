"""The product's host sampler / accept-prefix (C ABI) against the reference's golden vectors and
against the Python oracle on seeded random rows.  No GPU needed."""
import math
import os
import struct
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle"))
import sampling as S  # noqa: E402
from dflb import pkg  # noqa: E402

NAN = float("nan")
VOCAB = 6
INPUT = [0, 1, 2, 3]


def f64_bits(x):
    return struct.unpack("<Q", struct.pack("<d", x))[0]


def test_golden_rng_vectors_and_sample_stream():
    # crates/qwen-llm/src/sampling.rs:1817-1878
    assert pkg.splitmix64_stream(0, 4) == [0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4, 0x06C45D188009454F, 0xF88BB8A8724C81EC]
    s = pkg.Sampler(temperature=1.0, seed=0x123456789ABCDEF0)
    assert [s.next_u64() for _ in range(4)] == [0x4D4F7607A97A1BD6, 0x9BA027C76910D021, 0x87ADB062153AE0BC, 0xB750F7B1FF944783]
    s = pkg.Sampler(temperature=1.0, seed=0)
    assert [f64_bits(s.next_unit_f64()) for _ in range(4)] == [0x3FD4C5D7585242C8, 0x3FD8769BCF70E034, 0x3FD703F7E47B269E, 0x3F8775FC61DDF2C0]
    s = pkg.Sampler(temperature=1.0, seed=0x123456789ABCDEF0)
    assert [s.sample([2.0, 1.5, 1.0, 0.5])[0] for _ in range(16)] == [0, 1, 1, 1, 3, 1, 3, 0, 0, 3, 0, 0, 2, 0, 2, 1]


def test_greedy_ties_and_errors():
    assert pkg.greedy_token([1.0, 5.0, 5.0, 3.0]) == 1
    assert pkg.greedy_token([-0.0, 0.0, -0.0]) == 1
    assert pkg.greedy_token([0.0, -0.0, 0.0]) == 0
    for kw in (dict(temperature=NAN), dict(temperature=-1.0), dict(top_p=0.0), dict(top_p=1.1), dict(min_p=-0.1), dict(min_p=1.1)):
        with pytest.raises(pkg.DflError):
            pkg.Sampler(**kw)
    s = pkg.Sampler()
    with pytest.raises(pkg.DflError):
        s.sample(np.zeros(0, dtype=np.float32))
    with pytest.raises(pkg.DflError) as e:
        s.sample([0.0, NAN])
    assert "token 1" in str(e.value)


@pytest.mark.parametrize("cfg", [dict(temperature=0.7, top_p=0.95), dict(temperature=1.0), dict(temperature=0.7, top_k=200, min_p=0.05),
                                 dict(temperature=1.3, top_k=20, top_p=0.9, min_p=0.01), dict(temperature=0.0)])
def test_sample_stream_equals_oracle_on_random_rows(cfg):
    rng = np.random.default_rng(42)
    prod = pkg.Sampler(seed=99, **cfg)
    orc_s = S.Sampler(S.SamplingConfig(seed=99, **cfg))
    for it in range(12):
        v = int(rng.integers(50, 4000))
        row = (rng.standard_normal(v) * 3).astype(np.float32)
        if it % 3 == 0:
            row[rng.integers(0, v, 5)] = row.max()        # ties at the top
        if it % 4 == 1:
            row[rng.integers(0, v, 3)] = -np.inf
        assert prod.sample(row) == orc_s.sample([float(x) for x in row])
        assert prod.draws == orc_s.draws
    assert prod.rng_state() == orc_s.rng.state


def test_sparse_coupling_equals_oracle():
    rng = np.random.default_rng(7)
    for seed in range(40):
        cfg = dict(temperature=0.7, top_k=0, top_p=0.95, min_p=0.0)
        prod = pkg.Sampler(seed=seed, **cfg)
        o = S.Sampler(S.SamplingConfig(seed=seed, **cfg))
        v = 300
        row = (rng.standard_normal(v) * 2).astype(np.float32)
        top = np.argsort(-row)[:16]
        cands = [(int(t), float(math.exp(row[t] / 0.7))) for t in top]
        tok = int(top[rng.integers(0, 4)])
        assert prod.couple_sparse(row, tok, cands) == o.couple_sparse_proposal([float(x) for x in row], S.SparseProposal(tok, cands))
        assert prod.rng_state() == o.rng.state and prod.draws == o.draws


# ---- accept.rs tests through the C ABI ----------------------------------------------------
def sampler(temperature):
    return pkg.Sampler(temperature=temperature, top_k=1, seed=17)


def logits(winners):
    v = [-10.0] * (len(winners) * VOCAB)
    for row, tok in enumerate(winners):
        v[row * VOCAB + tok] = 10.0
    return v


def one_hot():
    return [(t, [(t, 1.0)]) for t in INPUT[1:]]


def same_rng(s, draws, temperature=1.0):
    ref = pkg.Sampler(temperature=temperature, top_k=1, seed=17, at_draw=draws)
    return s.draws == draws and s.rng_state() == ref.rng_state()


def test_every_rejection_position():
    for temperature in (0.0, 1.0):
        for sparse in (False, True):
            for rejected_row in range(3):
                winners = [1, 2, 3, 4]
                winners[rejected_row] = 5
                rows = logits(winners)
                for i in range((rejected_row + 1) * VOCAB, len(rows)):
                    rows[i] = NAN
                req = sampler(temperature)
                d = pkg.accept_prefix(INPUT, rows, VOCAB, one_hot() if sparse else None, req, 4, [])
                assert d["accepted_drafts"] == INPUT[1:1 + rejected_row]
                assert d["next_carry"] == ("correction", 5) and d["stop_reason"] is None
                assert d["retain_input_count"] == 1 + rejected_row
                draws = rejected_row + 2 if sparse else (rejected_row + 1 if temperature > 0 else 0)
                assert same_rng(req, draws, temperature)


def test_all_accepted_bonus_eos_cap_anchor():
    for temperature in (0.0, 1.0):
        for sparse in (False, True):
            req = sampler(temperature)
            d = pkg.accept_prefix(INPUT, logits([1, 2, 3, 4]), VOCAB, one_hot() if sparse else None, req, 4, [])
            assert (d["accepted_drafts"], d["next_carry"], d["stop_reason"], d["retain_input_count"]) == ([1, 2, 3], ("bonus", 4), None, 4)
            assert same_rng(req, 4 if temperature > 0 else (3 if sparse else 0), temperature)
    for sparse in (False, True):
        for terminal_count in (1, 2, 3):
            for eos, cap in ((True, False), (False, True), (True, True)):
                rows = logits([1, 2, 3, 4])
                for i in range(terminal_count * VOCAB, len(rows)):
                    rows[i] = NAN
                props = one_hot()
                for j in range(terminal_count, 3):
                    props[j] = (props[j][0], [(props[j][0], NAN)])
                req = sampler(1.0)
                d = pkg.accept_prefix(INPUT, rows, VOCAB, props if sparse else None, req, terminal_count if cap else 4,
                                      [INPUT[terminal_count]] if eos else [])
                assert d["accepted_drafts"] == INPUT[1:terminal_count + 1] and d["next_carry"] is None
                assert d["stop_reason"] == ("eos" if eos else "token_limit") and d["retain_input_count"] == terminal_count
                assert same_rng(req, terminal_count)
    for inp in (INPUT[:1], INPUT):
        for budget, stops, reason in ((0, [], "token_limit"), (0, [0], "eos"), (4, [0], "eos")):
            req = sampler(1.0)
            d = pkg.accept_prefix(inp, [NAN] * (len(inp) * VOCAB), VOCAB, None, req, budget, stops)
            assert (d["accepted_drafts"], d["next_carry"], d["stop_reason"], d["retain_input_count"]) == ([], None, reason, 0)
            assert same_rng(req, 0)
    for props in (None, []):
        req = sampler(1.0)
        d = pkg.accept_prefix([0], logits([4]), VOCAB, props, req, 1, [4])
        assert (d["accepted_drafts"], d["next_carry"], d["retain_input_count"]) == ([], ("bonus", 4), 1) and req.draws == 1
    d = pkg.accept_prefix(INPUT, logits([5, 2, 3, 4]), VOCAB, None, sampler(1.0), 1, [5])
    assert (d["accepted_drafts"], d["next_carry"], d["retain_input_count"]) == ([], ("correction", 5), 1)


def test_errors_leave_rng_unchanged():
    rows = logits([1, 2, 3, 4])
    props = one_hot()
    mismatch = one_hot()
    mismatch[2] = (4, mismatch[2][1])
    bad_cand = one_hot()
    bad_cand[2] = (3, [(-1, 1.0)])
    cases = [([], [], VOCAB, None), (INPUT, rows, 0, None), (INPUT, rows, 1 << 63, None), (INPUT, rows[:-1], VOCAB, None),
             (INPUT[:3], rows, VOCAB, None), ([-1, 1, 2, 3], rows, VOCAB, None), ([0, 1, 2, 6], rows, VOCAB, None),
             (INPUT, rows, VOCAB, props[:2]), (INPUT, rows, VOCAB, mismatch), (INPUT, rows, VOCAB, bad_cand)]
    for inp, r, vocab, p in cases:
        for budget in (0, 4):
            req = sampler(1.0)
            with pytest.raises(pkg.DflError):
                pkg.accept_prefix(inp, r, vocab, p, req, budget, [])
            assert same_rng(req, 0)
    for row in (1, 2, 3):
        rows = logits([1, 2, 3, 4])
        rows[row * VOCAB] = NAN
        req = sampler(1.0)
        with pytest.raises(pkg.DflError) as e:
            pkg.accept_prefix(INPUT, rows, VOCAB, None, req, 4, [])
        assert f"row {row}" in str(e.value)
        assert same_rng(req, 0)
    rows = logits([1, 2, 3, 4])
    for invalid in ((2, []), (2, [(2, -1.0)]), (2, [(2, NAN)]), (2, [(2, 0.0)]), (2, [(1, 1.0)])):
        props = one_hot()
        props[1] = invalid
        req = sampler(1.0)
        with pytest.raises(pkg.DflError) as e:
            pkg.accept_prefix(INPUT, rows, VOCAB, props, req, 4, [])
        assert "row 1" in str(e.value)
        assert same_rng(req, 0)


def test_accept_prefix_equals_oracle_on_random_blocks():
    rng = np.random.default_rng(11)
    v = 500
    for it in range(30):
        n = int(rng.integers(1, 17))
        rows = (rng.standard_normal((n, v)) * 4).astype(np.float32)
        verified = [int(rng.integers(0, v))]
        for r in range(n - 1):
            verified.append(int(np.argmax(rows[r])) if rng.random() < 0.6 else int(rng.integers(0, v)))
        cfg = dict(temperature=0.7, top_p=0.95) if it % 2 else dict(temperature=0.0)
        prod = pkg.Sampler(seed=it, **cfg)
        o = S.Sampler(S.SamplingConfig(seed=it, **cfg))
        d = pkg.accept_prefix(verified, rows, v, None, prod, 100, [])
        w = S.decide_dflash_accept_prefix(verified, [float(x) for x in rows.reshape(-1)], v, None, o, 100, [])
        assert d["accepted_drafts"] == w.accepted_drafts and d["next_carry"] == w.next_carry
        assert d["retain_input_count"] == w.retain_input_count and prod.draws == o.draws and prod.rng_state() == o.rng.state


def test_rows_prepared_ahead_on_large_vocab_equal_oracle_and_keep_error_rows():
    """At vocabularies of 4096 and more the product builds every row's distribution ahead of the sequential accept loop
    on host threads; decisions, draw counts, generator state and error rows must not change."""
    rng = np.random.default_rng(21)
    v = 4608
    for it in range(6):
        n = 16 if it < 4 else int(rng.integers(2, 17))
        rows = (rng.standard_normal((n, v)) * 5).astype(np.float32)
        rows[:, :8] += 14.0            # a few dominant tokens so that drafts get accepted
        verified = [int(rng.integers(0, v))]
        for r in range(n - 1):
            verified.append(int(np.argmax(rows[r])) if rng.random() < 0.7 else int(rng.integers(0, v)))
        cfg = dict(temperature=0.7, top_p=0.95)
        sparse = None
        if it % 2:    # sparse proposals: the draft plus one other candidate
            sparse = [(verified[r + 1], [(verified[r + 1], 0.75), ((verified[r + 1] + 1) % v, 0.25)]) for r in range(n - 1)]
        prod = pkg.Sampler(seed=it, **cfg)
        o = S.Sampler(S.SamplingConfig(seed=it, **cfg))
        d = pkg.accept_prefix(verified, rows, v, sparse, prod, 100, [])
        osparse = None if sparse is None else [S.SparseProposal(t, c) for t, c in sparse]
        w = S.decide_dflash_accept_prefix(verified, [float(x) for x in rows.reshape(-1)], v, osparse, o, 100, [])
        assert d["accepted_drafts"] == w.accepted_drafts and d["next_carry"] == w.next_carry
        assert prod.draws == o.draws and prod.rng_state() == o.rng.state
    # a NaN in a row the loop never reaches is not an error; in a reached row it is, with the generator untouched
    rows = np.zeros((4, v), dtype=np.float32)
    rows[:, 3] = 50.0                   # every row samples token 3
    verified = [0, 3, 9, 3]             # row 1's draft (9) is rejected
    rows[2, 100] = NAN
    req = pkg.Sampler(temperature=1.0, seed=5)
    d = pkg.accept_prefix(verified, rows, v, None, req, 100, [])
    assert d["accepted_drafts"] == [3] and d["next_carry"] == ("correction", 3) and req.draws == 2
    rows[2, 100] = 0.0
    rows[1, 100] = NAN
    req = pkg.Sampler(temperature=1.0, seed=5)
    before = req.rng_state()
    with pytest.raises(pkg.DflError) as e:
        pkg.accept_prefix(verified, rows, v, None, req, 100, [])
    assert "row 1" in str(e.value) and req.rng_state() == before and req.draws == 0
