"""DFlash 2 path selector on the host: the Python oracle and the product's C ABI against the reference's own
selector tests (crates/qwen-llm/src/metal_dflash/tests.rs:2797-3095), then against each other on seeded inputs.
No GPU needed."""
import math
import os
import struct
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle"))
import sampling as S  # noqa: E402
import selector as SEL  # noqa: E402
import orc  # noqa: E402
from dflb import pkg  # noqa: E402

INF, NAN = float("inf"), float("nan")


def f32_codebook_bytes(rows):
    return np.asarray(rows, dtype=np.float32).tobytes()


def both_codebooks(dtype, rank, n_rows, raw):
    return SEL.Codebook(dtype, rank, n_rows, raw), pkg.Codebook(dtype, rank, n_rows, raw)


def test_legacy_codebook_formats_preserve_row_boundaries():
    # tests.rs:2862-2957: [3, 2] F32 / F16 / BF16 codebooks, row 1; [32, 2] Q8_0, row 1
    values = [1.0, -2.0, 3.5, 4.25, -5.5, 6.75]
    for dtype, raw in ((SEL.F32, np.asarray(values, np.float32).tobytes()), (SEL.F16, np.asarray(values, np.float16).tobytes()),
                       (SEL.BF16, (np.asarray(values, np.float32).view(np.uint32) >> 16).astype(np.uint16).tobytes())):
        for cb in both_codebooks(dtype, 3, 2, raw):
            assert cb.dequant_row(1).tolist() == [4.25, -5.5, 6.75]
    q8 = bytearray(68)
    for row in range(2):
        q8[34 * row:34 * row + 2] = np.float16(0.25 * (row + 1)).tobytes()
        for i in range(32):
            q8[34 * row + 2 + i] = (i - 12 + row) & 0xFF
    for cb in both_codebooks(SEL.Q8_0, 32, 2, bytes(q8)):
        assert cb.dequant_row(1).tolist() == [0.5 * (i - 11.0) for i in range(32)]


def test_q4_k_codebook_rows_match_whole_tensor_dequant():
    # tests.rs:2797-2822: every row of a [256, n] Q4_K codebook equals that slice of the whole tensor's dequantisation
    rng = np.random.default_rng(5)
    w = (rng.standard_normal((5, 256)) * 0.3).astype(np.float32)
    raw = bytes(orc.quantize(orc.Q4_K, w))
    whole = orc.dequant(orc.Q4_K, np.frombuffer(raw, dtype=np.uint8), 5 * 256).reshape(5, 256)
    for cb in both_codebooks(SEL.Q4_K, 256, 5, raw):
        for row in range(5):
            assert np.array_equal(cb.dequant_row(row).view(np.uint32), whole[row].view(np.uint32))


def test_codebook_rejects_bad_geometry_and_payloads():
    # tests.rs:2825-2859
    raw = bytes(144 * 2)
    for make in (SEL.Codebook, pkg.Codebook):
        with pytest.raises((ValueError, pkg.DflError)):
            make(SEL.Q4_K, 512, 1, bytes(288))       # Q4_K rank must be 256
        with pytest.raises((ValueError, pkg.DflError)):
            make(SEL.Q4_K, 256, 2, raw[:-1])          # truncated payload
        with pytest.raises((ValueError, pkg.DflError)):
            make(SEL.Q4_K, 256, 2, raw + b"\0")       # trailing byte
        with pytest.raises((ValueError, pkg.DflError)):
            make(SEL.Q8_0, 48, 1, bytes(51))          # rank not block-aligned
        with pytest.raises((ValueError, pkg.DflError)):
            make(14, 256, 1, bytes(210))              # Q6_K is not a codebook dtype
        cb = make(SEL.Q4_K, 256, 2, raw)
        with pytest.raises((IndexError, pkg.DflError)):
            cb.dequant_row(2)


def selector_test_codebooks(pred_rows, succ_rows):
    rank = len(pred_rows[0])
    o = (SEL.Codebook(SEL.F32, rank, len(pred_rows), f32_codebook_bytes(pred_rows)),
         SEL.Codebook(SEL.F32, rank, len(succ_rows), f32_codebook_bytes(succ_rows)))
    p = (pkg.Codebook(SEL.F32, rank, len(pred_rows), f32_codebook_bytes(pred_rows)),
         pkg.Codebook(SEL.F32, rank, len(succ_rows), f32_codebook_bytes(succ_rows)))
    return o, p


def walk_both(o, p, top_k, rank, carry, n, ids, unary, gates):
    """oracle and product walks in one shape: tokens, per-depth scores with None for unscored candidates, chosen index"""
    t_o, sc_o, ch_o = SEL.walk_greedy(o[0], o[1], top_k, rank, carry, n, ids, unary, gates)
    t_p, sc_p, scored = pkg.selector_walk(p[0], p[1], top_k, rank, carry, n, ids, unary, gates)
    sc_p = [[float(sc_p[d, b]) if scored[d, b] else None for b in range(top_k)] for d in range(1, n)]
    sc_o = [[None if x is None else float(x) for x in row] for row in sc_o]
    return (list(t_o), sc_o, ch_o), (t_p.tolist(), sc_p)


def same(a, b):
    return (a is None and b is None) or (a is not None and b is not None and (a == b or (math.isnan(a) and math.isnan(b))))


def test_selector_scores_and_tracks_predecessors():
    # tests.rs:2978-2997
    o, p = selector_test_codebooks([[1.0, 2.0], [2.0, 0.0], [0.0, 3.0], [1.0, 1.0]], [[0.0, 0.0], [1.0, 1.0], [2.0, 0.0], [0.0, 1.0]])
    (t_o, sc_o, ch_o), (t_p, sc_p) = walk_both(o, p, 2, 2, 0, 3, [0, 0, 1, 2, 3, 1], [0.0] * 6, [0.0, 0.0, 2.0, 0.5, 1.0, 2.0])
    assert t_o == [0, 2, 3] and t_p == [0, 2, 3]
    assert sc_o == [[3.0, 4.0], [6.0, 6.0]] and sc_p == sc_o
    assert ch_o == [1, 0]


def test_selector_keeps_first_tie_and_skips_sentinels():
    # tests.rs:2999-3027: duplicate ids both score, -1 and out-of-range ids are not scored, the first of a tie wins
    o, p = selector_test_codebooks([[1.0], [1.0]], [[0.0], [1.0]])
    (t_o, sc_o, ch_o), (t_p, sc_p) = walk_both(o, p, 4, 1, 0, 2, [0, 0, 0, 0, 1, 1, -1, 9], [0.0] * 8, [0.0, 1.0])
    assert ch_o == [0] and t_o[1] == 1 and t_p[1] == 1
    assert sc_o == [[1.0, 1.0, None, None]] and sc_p == sc_o


def test_selector_nonfinite_scores_and_no_valid_choice():
    # tests.rs:3029-3062: +inf wins; NaN and -inf never beat the initial -inf, so slot 0 is the fallback
    o, p = selector_test_codebooks([[1.0], [1.0], [1.0]], [[0.0], [0.0], [0.0]])
    (t_o, sc_o, ch_o), (t_p, sc_p) = walk_both(o, p, 2, 1, 0, 3, [0, 0, 1, 2, 1, 2], [0.0, 0.0, INF, 0.0, NAN, -INF], [0.0, 1.0, 1.0])
    assert ch_o == [0, 0]
    assert t_o == [0, 1, 1] and t_p == [0, 1, 1]
    assert sc_o[0] == [INF, 0.0] and math.isnan(sc_o[1][0]) and sc_o[1][1] == -INF
    assert all(same(a, b) for ra, rb in zip(sc_o, sc_p) for a, b in zip(ra, rb))


def test_selector_walk_rejects_invalid_predecessor_and_bad_lengths():
    # tests.rs:3076-3095: the chosen token (2) has no predecessor row; :3494-3512: length checks
    o, p = selector_test_codebooks([[1.0], [1.0]], [[0.0], [0.0], [1.0]])
    with pytest.raises(IndexError):
        SEL.walk_greedy(o[0], o[1], 1, 1, 0, 2, [0, 2], [0.0, 1.0], [0.0, 1.0])
    with pytest.raises(pkg.DflError) as e:
        pkg.selector_walk(p[0], p[1], 1, 1, 0, 2, [0, 2], [0.0, 1.0], [0.0, 1.0])
    assert "row out of range" in str(e.value)
    with pytest.raises(pkg.DflError):
        pkg.selector_walk(p[0], p[1], 1, 1, 0, 2, [0, 2, 1], [0.0, 1.0], [0.0, 1.0])
    with pytest.raises(pkg.DflError):
        pkg.selector_walk(p[0], p[1], 0, 1, 0, 2, [], [], [0.0, 1.0])


def random_selector_case(seed, dtype, vocab=300, rank=256, n=16):
    rng = np.random.default_rng(seed)
    books = []
    for _ in range(2):
        w = (rng.standard_normal((vocab, rank)) * 0.5).astype(np.float32)
        raw = bytes(orc.quantize(dtype, w)) if dtype in (orc.Q4_K, orc.Q8_0) else (
            w.tobytes() if dtype == SEL.F32 else w.astype(np.float16).tobytes() if dtype == SEL.F16 else
            (w.view(np.uint32) >> 16).astype(np.uint16).tobytes())
        books.append(raw)
    ids = np.stack([rng.permutation(vocab)[:16] for _ in range(n)]).astype(np.int32)
    vals = -np.sort(-rng.standard_normal((n, 16)).astype(np.float32) * 2.0, axis=1)
    ids[3, 14:] = -1                      # a short row's sentinels
    vals[3, 14:] = -np.inf
    sel_h = (rng.standard_normal((n, rank)) * 0.3).astype(np.float32)
    carry = int(rng.integers(0, vocab))
    return books, ids, vals, sel_h, carry


@pytest.mark.parametrize("dtype", [SEL.F32, SEL.F16, SEL.BF16, SEL.Q8_0, SEL.Q4_K])
def test_product_walk_equals_oracle_walk_on_seeded_blocks(dtype):
    for seed in range(4):
        books, ids, vals, sel_h, carry = random_selector_case(100 + seed, dtype)
        o = [SEL.Codebook(dtype, 256, 300, b) for b in books]
        p = [pkg.Codebook(dtype, 256, 300, b) for b in books]
        t_o, sc_o, _ = SEL.walk_greedy(o[0], o[1], 16, 256, carry, 16, ids, vals, sel_h)
        t_p, sc_p, scored = pkg.selector_walk(p[0], p[1], 16, 256, carry, 16, ids, vals, sel_h)
        assert t_p.tolist() == t_o
        for d in range(1, 16):
            for b in range(16):
                if sc_o[d - 1][b] is None:
                    assert not scored[d, b]
                else:   # same f32 operations in the same order: bit-equal
                    assert scored[d, b] and np.float32(sc_o[d - 1][b]).view(np.uint32) == sc_p[d, b].view(np.uint32)


def test_sampled_walk_equals_oracle_and_leaves_sampler_untouched_on_error():
    books, ids, vals, sel_h, carry = random_selector_case(7, SEL.Q8_0)
    o = [SEL.Codebook(SEL.Q8_0, 256, 300, b) for b in books]
    p = [pkg.Codebook(SEL.Q8_0, 256, 300, b) for b in books]
    so = S.Sampler(S.SamplingConfig(temperature=0.7, seed=0x44464C4153483251))
    sp = pkg.Sampler(temperature=0.7, seed=0x44464C4153483251)
    for _ in range(3):    # three blocks from one sampler stream
        t_o, pr_o = SEL.walk_sampled(o[0], o[1], 16, 256, carry, 16, ids, vals, sel_h, so)
        t_p, pr_p = pkg.selector_walk_sampled(p[0], p[1], 16, 256, carry, 16, ids, vals, sel_h, sp)
        assert t_p.tolist()[1:] == t_o[1:]
        assert len(pr_o) == len(pr_p) == 15
        for (tok_o, c_o), (tok_p, c_p) in zip(pr_o, pr_p):
            assert tok_o == tok_p and [c[0] for c in c_o] == [c[0] for c in c_p]
            assert [struct.pack("<d", c[1]) for c in c_o] == [struct.pack("<d", c[1]) for c in c_p]   # f64 weights bit-equal
        assert sp.draws == so.draws
        carry = t_o[-1]
    # a proposal sampler with a target-side filter is refused before any draw (metal_dflash.rs:17279-17288)
    bad = pkg.Sampler(temperature=0.7, top_p=0.9, seed=1)
    with pytest.raises(pkg.DflError):
        pkg.selector_walk_sampled(p[0], p[1], 16, 256, carry, 16, ids, vals, sel_h, bad)
    assert bad.draws == 0
    with pytest.raises(ValueError):
        SEL.walk_sampled(o[0], o[1], 16, 256, carry, 16, ids, vals, sel_h, S.Sampler(S.SamplingConfig(temperature=0.7, top_p=0.9, seed=1)))


def test_oracle_topk16_order_ties_and_sentinels():
    # kernels/dflash2.metal:69-84: total order (so +0 > -0, NaN above +inf by sign), ties to the lower index
    x = np.zeros((3, 40), dtype=np.float32)
    x[0] = np.arange(40) % 7          # many ties: lowest indices first within a value
    x[1, :] = -1.0
    x[1, 5], x[1, 9], x[1, 11] = 0.0, -0.0, np.nan
    x[2, :] = np.float32(-np.inf)
    x[2, 3] = np.frombuffer(struct.pack("<I", 0xFFC00000), dtype=np.float32)[0]   # negative NaN: below -inf, never listed
    ids, vals = SEL.topk16(x)
    assert ids[0].tolist() == [6, 13, 20, 27, 34, 5, 12, 19, 26, 33, 4, 11, 18, 25, 32, 39]
    assert ids[1].tolist()[:3] == [11, 5, 9] and ids[1].tolist()[3:] == [i for i in range(40) if i not in (5, 9, 11)][:13]
    assert 3 not in ids[2].tolist() and ids[2].tolist() == [i for i in range(40) if i != 3][:16]
    short = SEL.topk16(np.asarray([[1.0, 3.0, 2.0]], dtype=np.float32))
    assert short[0][0].tolist() == [1, 2, 0] + [-1] * 13 and np.all(np.isneginf(short[1][0][3:]))
