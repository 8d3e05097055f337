"""Pins the Python sampler / accept-prefix oracle to the reference's golden vectors
(crates/qwen-llm/src/sampling.rs:1817-1878, :1790-1796, :1904-1930) and restates its
accept-prefix tests (crates/qwen-llm/src/metal_dflash/accept.rs:236-616) in meaning."""
import math
import os
import struct
import sys

import pytest

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle"))
import sampling as S  # noqa: E402

NAN = float("nan")
VOCAB = 6
INPUT = [0, 1, 2, 3]


def f64_bits(x):
    return struct.unpack("<Q", struct.pack("<d", x))[0]


def test_rng_and_sample_stream_match_version_one_golden_vectors():
    sm = S.SplitMix64(0)
    assert [sm.next() for _ in range(4)] == [0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4, 0x06C45D188009454F, 0xF88BB8A8724C81EC]
    rng = S.Xoshiro256PlusPlus(0x123456789ABCDEF0)
    assert [rng.next_u64() for _ in range(4)] == [0x4D4F7607A97A1BD6, 0x9BA027C76910D021, 0x87ADB062153AE0BC, 0xB750F7B1FF944783]
    rng = S.Xoshiro256PlusPlus(0)
    assert [f64_bits(rng.next_unit_f64()) for _ in range(4)] == [0x3FD4C5D7585242C8, 0x3FD8769BCF70E034, 0x3FD703F7E47B269E, 0x3F8775FC61DDF2C0]
    s = S.Sampler(S.SamplingConfig(temperature=1.0, seed=0x123456789ABCDEF0))
    assert [s.sample([2.0, 1.5, 1.0, 0.5])[0] for _ in range(16)] == [0, 1, 1, 1, 3, 1, 3, 0, 0, 3, 0, 0, 2, 0, 2, 1]


def test_greedy_ties_and_signed_zero():
    assert S.greedy_token([1.0, 5.0, 5.0, 3.0]) == 1
    assert S.greedy_token([2.0, 2.0, 2.0]) == 0
    assert S.greedy_token([-0.0, 0.0, -0.0]) == 1
    assert S.greedy_token([0.0, -0.0, 0.0]) == 0
    assert S.Sampler(S.SamplingConfig()).sample([1.0, 3.0, 3.0])[0] == 1


def test_invalid_configuration_and_logits():
    for kw in (dict(temperature=NAN), dict(temperature=-1.0), dict(temperature=math.inf), dict(top_p=0.0),
               dict(top_p=-0.1), dict(top_p=1.1), dict(min_p=-0.1), dict(min_p=1.1), dict(min_p=math.inf)):
        with pytest.raises(S.SamplingError):
            S.Sampler(S.SamplingConfig(**kw))
    s = S.Sampler(S.SamplingConfig())
    with pytest.raises(S.SamplingError):
        s.sample([])
    with pytest.raises(S.SamplingError) as e:
        s.sample([0.0, NAN])
    assert e.value.kind == "NanLogit" and e.value.detail == 1


def test_top_k_one_forces_argmax_and_consumes_one_draw():
    s = S.Sampler(S.SamplingConfig(temperature=1.0, top_k=1, seed=7))
    for draw in range(1, 33):
        assert s.sample([0.0, 3.0, 1.0])[0] == 1
        assert s.draws == draw


def test_draw_count_reconstructs_stream():
    cfg = S.SamplingConfig(temperature=1.0, seed=7)
    a = S.Sampler(cfg)
    logits = [1.0, 0.5, 0.0]
    for _ in range(17):
        a.sample(logits)
    b = S.Sampler.at_draw(cfg, a.draws)
    for _ in range(32):
        assert a.sample(logits) == b.sample(logits)


# ---- accept.rs tests ------------------------------------------------------
def sampler(temperature):
    return S.Sampler(S.SamplingConfig(temperature=temperature, top_k=1, seed=17))


def logits(winners):
    v = [-10.0] * (len(winners) * VOCAB)
    for row, tok in enumerate(winners):
        v[row * VOCAB + tok] = 10.0
    return v


def one_hot():
    return [S.SparseProposal(t, [(t, 1.0)]) for t in INPUT[1:]]


def same_rng(a, b):
    return a.draws == b.draws and a.rng.state == b.rng.state


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
                d = S.decide_dflash_accept_prefix(INPUT, rows, VOCAB, one_hot() if sparse else None, req, 4, [])
                assert d.accepted_drafts == INPUT[1:1 + rejected_row]
                assert d.next_carry == ("correction", 5)
                assert d.stop_reason is None and d.retain_input_count == 1 + rejected_row
                draws = rejected_row + 2 if sparse else (rejected_row + 1 if temperature > 0 else 0)
                assert same_rng(req, S.Sampler.at_draw(req.config, draws))


def test_all_accepted_samples_bonus():
    for temperature in (0.0, 1.0):
        for sparse in (False, True):
            req = sampler(temperature)
            d = S.decide_dflash_accept_prefix(INPUT, logits([1, 2, 3, 4]), VOCAB, one_hot() if sparse else None, req, 4, [])
            assert (d.accepted_drafts, d.next_carry, d.stop_reason, d.retain_input_count) == ([1, 2, 3], ("bonus", 4), None, 4)
            draws = 4 if temperature > 0 else (3 if sparse else 0)
            assert same_rng(req, S.Sampler.at_draw(req.config, draws))


def test_eos_and_cap_leave_terminal_unconsumed():
    for sparse in (False, True):
        for terminal_count in (1, 2, 3):
            for eos, cap in ((True, False), (False, True), (True, True)):
                rows = logits([1, 2, 3, 4])
                for i in range(terminal_count * VOCAB, len(rows)):
                    rows[i] = NAN
                props = one_hot()
                for tail in props[terminal_count:]:
                    tail.candidates[0] = (tail.candidates[0][0], NAN)
                stops = [INPUT[terminal_count]] if eos else []
                req = sampler(1.0)
                d = S.decide_dflash_accept_prefix(INPUT, rows, VOCAB, props if sparse else None, req,
                                                  terminal_count if cap else 4, stops)
                assert d.accepted_drafts == INPUT[1:terminal_count + 1]
                assert d.next_carry is None
                assert d.stop_reason == ("eos" if eos else "token_limit")
                assert d.retain_input_count == terminal_count
                assert same_rng(req, S.Sampler.at_draw(req.config, terminal_count))


def test_terminal_anchor_and_zero_budget():
    for inp in (INPUT[:1], INPUT):
        for budget, stops, reason in ((0, [], "token_limit"), (0, [0], "eos"), (4, [0], "eos")):
            req = sampler(1.0)
            before = req.clone()
            d = S.decide_dflash_accept_prefix(inp, [NAN] * (len(inp) * VOCAB), VOCAB, None, req, budget, stops)
            assert (d.accepted_drafts, d.next_carry, d.stop_reason, d.retain_input_count) == ([], None, reason, 0)
            assert same_rng(req, before)


def test_anchor_only_bonus_and_rejection_carry():
    for props in (None, []):
        req = sampler(1.0)
        d = S.decide_dflash_accept_prefix([0], logits([4]), VOCAB, props, req, 1, [4])
        assert (d.accepted_drafts, d.next_carry, d.stop_reason, d.retain_input_count) == ([], ("bonus", 4), None, 1)
        assert req.draws == 1
    d = S.decide_dflash_accept_prefix(INPUT, logits([5, 2, 3, 4]), VOCAB, None, sampler(1.0), 1, [5])
    assert (d.accepted_drafts, d.next_carry, d.stop_reason, d.retain_input_count) == ([], ("correction", 5), None, 1)


def test_sparse_coupling_uses_actual_q_and_target_filters():
    target_row = [2.0, 1.9, 1.5, 0.5, -1.0, -2.0]
    rows = target_row + logits([4])
    high_q = S.SparseProposal(0, [(0, 8.0), (1, 1.0), (5, 1.0)])
    low_q = S.SparseProposal(0, [(0, 1.0), (1, 99.0)])
    accepted = rejected = 0
    for seed in range(64):
        cfg = S.SamplingConfig(temperature=0.7, top_k=4, top_p=0.7, min_p=0.5, seed=seed)
        req = S.Sampler(cfg)
        ref = req.clone()
        dec = ref.couple_sparse_proposal(target_row, high_q)
        if dec[0] == "accepted":
            accepted += 1
            expected = ([0], ("bonus", ref.sample(rows[VOCAB:])[0]), None, 2)
        else:
            rejected += 1
            assert dec[1] == 1
            expected = ([], ("correction", dec[1]), None, 1)
        d = S.decide_dflash_accept_prefix([3, 0], rows, VOCAB, [high_q], req, 2, [])
        assert (d.accepted_drafts, d.next_carry, d.stop_reason, d.retain_input_count) == expected
        assert same_rng(req, ref)
        low = S.decide_dflash_accept_prefix([3, 0], rows, VOCAB, [low_q], S.Sampler(cfg), 2, [])
        assert low.accepted_drafts == [0]
        filt = S.SparseProposal(2, [(2, 1.0), (0, 99.0)])
        req = S.Sampler(cfg)
        f = S.decide_dflash_accept_prefix([3, 2], rows, VOCAB, [filt], req, 2, [])
        assert f.accepted_drafts == [] and f.next_carry[0] == "correction" and f.next_carry[1] in (0, 1)
        assert req.draws == 2
    assert accepted > 0 and rejected > 0


def test_malformed_inputs_leave_rng_unchanged():
    rows = logits([1, 2, 3, 4])
    props = one_hot()
    mismatch = one_hot()
    mismatch[2].token = 4
    bad_cand = one_hot()
    bad_cand[2].candidates[0] = (-1, 1.0)
    cases = [([], [], VOCAB, None), (INPUT, rows, 0, None), (INPUT, rows, 1 << 63, None), (INPUT, rows[:-1], VOCAB, None),
             (INPUT[:3], rows, VOCAB, None), ([-1, 1, 2, 3], rows, VOCAB, None), ([0, 1, 2, 6], rows, VOCAB, None),
             (INPUT, rows, VOCAB, props[:2]), (INPUT, rows, VOCAB, mismatch), (INPUT, rows, VOCAB, bad_cand)]
    for inp, r, vocab, p in cases:
        for budget in (0, 4):
            req = sampler(1.0)
            before = req.clone()
            with pytest.raises(S.AcceptError):
                S.decide_dflash_accept_prefix(inp, r, vocab, p, req, budget, [])
            assert same_rng(req, before)


def test_errors_after_accepted_rows_roll_back_rng():
    for row in (1, 2, 3):
        rows = logits([1, 2, 3, 4])
        rows[row * VOCAB] = NAN
        req = sampler(1.0)
        before = req.clone()
        with pytest.raises(S.AcceptError) as e:
            S.decide_dflash_accept_prefix(INPUT, rows, VOCAB, None, req, 4, [])
        assert e.value.kind == "Sampling" and e.value.row == row
        assert same_rng(req, before)
    rows = logits([1, 2, 3, 4])
    for invalid in (S.SparseProposal(2, []), S.SparseProposal(2, [(2, -1.0)]), S.SparseProposal(2, [(2, NAN)]),
                    S.SparseProposal(2, [(2, 0.0)]), S.SparseProposal(2, [(1, 1.0)])):
        props = one_hot()
        props[1] = invalid
        req = sampler(1.0)
        before = req.clone()
        with pytest.raises(S.AcceptError) as e:
            S.decide_dflash_accept_prefix(INPUT, rows, VOCAB, props, req, 4, [])
        assert e.value.kind == "Sampling" and e.value.row == 1
        assert same_rng(req, before)
