"""GPU parity of the few-row quantised GEMM and the argmax kernel against the CPU oracle.
All calls go through the C ABI (dfl_qmatrix_*, dfl_fewrow_matmul, dfl_argmax_top2)."""
import numpy as np
import pytest

import orc
from dflb import pkg

pytestmark = pytest.mark.gpu

DTYPES = [(orc.Q4_K, "q4_k"), (orc.Q5_K, "q5_k"), (orc.Q6_K, "q6_k"), (orc.Q8_0, "q8_0"), (orc.BF16, "bf16")]


def make_weight(dtype, n_in, n_out, seed):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((n_out, n_in)) * 0.02).astype(np.float32)
    raw = orc.quantize(dtype, w)
    return raw, orc.dequant(dtype, raw, n_in * n_out).reshape(n_out, n_in)


@pytest.mark.parametrize("dtype,name", DTYPES)
@pytest.mark.parametrize("n_in,n_out", [(256, 128), (1024, 200), (4096, 1000)])
def test_resident_tiles_decode_to_ggml_values(dtype, name, n_in, n_out):
    raw, wf = make_weight(dtype, n_in, n_out, 11)
    m = pkg.QMatrix(dtype, n_in, n_out, raw)
    got = m.dequant()
    assert got.tobytes() == wf.tobytes()
    m.close()


@pytest.mark.parametrize("dtype,name", DTYPES)
def test_one_hot_rows_reproduce_every_weight_exactly(dtype, name):
    # metal/tests/q6_k_f32_tile.rs:152-181: basis-vector inputs must return the decoded weights
    n_in, n_out = 512, 160
    raw, wf = make_weight(dtype, n_in, n_out, 3)
    m = pkg.QMatrix(dtype, n_in, n_out, raw)
    for base in range(0, n_in, 16):
        x = np.zeros((16, n_in), dtype=np.float32)
        for r in range(16):
            x[r, base + r] = 1.0
        y = m.matmul(x)
        want = wf[:, base:base + 16].T
        assert y.tobytes() == np.ascontiguousarray(want).tobytes(), f"columns {base}..{base + 15}"
    m.close()


@pytest.mark.parametrize("dtype,name", DTYPES)
@pytest.mark.parametrize("n_in,n_out,n_rows", [(256, 128, 1), (1024, 200, 5), (4096, 1000, 16), (12288, 384, 16)])
def test_matmul_matches_oracle(dtype, name, n_in, n_out, n_rows):
    raw, wf = make_weight(dtype, n_in, n_out, 5)
    rng = np.random.default_rng(17)
    x = rng.standard_normal((n_rows, n_in)).astype(np.float32)
    want = orc.matmul(dtype, raw, n_in, n_out, x)
    m = pkg.QMatrix(dtype, n_in, n_out, raw)
    got = m.matmul(x)
    # contract: 1e-2 relative + 1e-3 absolute; the kernel is far inside it
    np.testing.assert_allclose(got, want, rtol=1e-2, atol=1e-3)
    # f32 accumulation bound against an f64 product (q6_k_f32_tile.rs:190-255)
    exact = x.astype(np.float64) @ wf.astype(np.float64).T
    bound = (np.abs(x).astype(np.float64) @ np.abs(wf).astype(np.float64).T) * (n_in * 2.0 ** -24) + 1e-30
    assert np.all(np.abs(got - exact) <= bound)
    m.close()


@pytest.mark.parametrize("dtype,name", DTYPES)
def test_rows_do_not_depend_on_row_count(dtype, name):
    # q6_k_f32_tile.rs:261-312: bitwise the same row for any number of rows in the call
    n_in, n_out = 2048, 256
    raw, _ = make_weight(dtype, n_in, n_out, 9)
    x = np.random.default_rng(2).standard_normal((16, n_in)).astype(np.float32)
    m = pkg.QMatrix(dtype, n_in, n_out, raw)
    full = m.matmul(x)
    for n in (1, 3, 8):
        part = m.matmul(x[:n])
        assert part.tobytes() == full[:n].tobytes()
    again = m.matmul(x)
    assert again.tobytes() == full.tobytes()  # deterministic
    m.close()


def q8_0_bytes(q, d):
    """ggml Q8_0 rows from int8 codes q [n_out][n_in] and f16 block scales d [n_out][n_in / 32]"""
    n_out, n_in = q.shape
    blocks = np.zeros((n_out, n_in // 32, 34), dtype=np.uint8)
    blocks[:, :, :2] = np.ascontiguousarray(d.astype(np.float16)).view(np.uint8).reshape(n_out, n_in // 32, 2)
    blocks[:, :, 2:] = q.reshape(n_out, n_in // 32, 32).view(np.uint8)
    return blocks.reshape(-1)


@pytest.mark.parametrize("scales,engine", [([2.0 ** -24, 2.0 ** -20, 6.1e-5, 1e-3, 0.0371, 1.0], "tcgen05"), ([256.0, -256.0, 0.5, -3e-4], "tcgen05"),
                                           ([300.0, 1.0], "mma.sync"), ([float("inf"), 1.0], "mma.sync")])
def test_q8_0_scale_range_decides_the_engine_and_every_weight_stays_exact(scales, engine):
    """The tensor-memory kernel folds a block's f16 scale into its operand as an exact pair of halfs; that holds for
    subnormal scales and up to |d| = 256 (q * d inside the f16 range).  Matrices beyond it run the mma.sync kernel."""
    rng = np.random.default_rng(31)
    n_in, n_out = 512, 130
    q = rng.integers(-128, 128, size=(n_out, n_in), dtype=np.int8)
    q[0, :32] = -128
    q[1, :32] = 127
    d = rng.choice(np.array(scales, dtype=np.float16), size=(n_out, n_in // 32))
    m = pkg.QMatrix(orc.Q8_0, n_in, n_out, q8_0_bytes(q, d))
    assert m.engine == engine
    if not np.all(np.isfinite(d.astype(np.float32))):
        m.close()
        return
    wf = q.astype(np.float32) * np.repeat(d.astype(np.float32), 32, axis=1)
    assert m.dequant().tobytes() == wf.tobytes()
    for base in range(0, n_in, 16):
        x = np.zeros((16, n_in), dtype=np.float32)
        x[np.arange(16), base + np.arange(16)] = 1.0
        # value equality: a zero code under a negative scale decodes to -0.0, while a sum of products starts from +0.0
        assert np.array_equal(m.matmul(x), wf[:, base:base + 16].T), f"columns {base}..{base + 15}"
    x = rng.standard_normal((16, n_in)).astype(np.float32)
    exact = x.astype(np.float64) @ wf.astype(np.float64).T
    bound = (np.abs(x).astype(np.float64) @ np.abs(wf).astype(np.float64).T) * (n_in * 2.0 ** -24) + 1e-30
    assert np.all(np.abs(m.matmul(x) - exact) <= bound)
    m.close()


@pytest.mark.parametrize("dtype,name,n_in,n_out", [(orc.Q6_K, "q6_k", 4096, 151936), (orc.Q8_0, "q8_0", 4096, 32768), (orc.Q5_K, "q5_k", 4096, 32768),
                                                   (orc.Q4_K, "q4_k", 4096, 32768)])
def test_repeated_launches_on_a_large_cold_matrix_give_the_same_bits(dtype, name, n_in, n_out):
    """The weight ring's "stage landed" barriers are per unpacking group when the stage count is odd (Q5_K, Q6_K, Q8_0):
    bulk copies complete out of order, and on a shared barrier a group that ran ahead once took the other group's
    outstanding copy for its own - one wrong row tile in the first, cold launch on a matrix of this size."""
    rng = np.random.default_rng(7)
    blk = {orc.Q4_K: 144, orc.Q5_K: 176, orc.Q6_K: 210, orc.Q8_0: 272}[dtype]
    nb = n_out * (n_in // 256)
    b = rng.integers(0, 256, size=(nb, blk), dtype=np.uint8)
    d = np.full(nb, 1e-4, dtype=np.float16).view(np.uint8).reshape(nb, 2)   # sane f16 block scales over random codes
    if dtype == orc.Q6_K:
        b[:, 208:210] = d
    elif dtype == orc.Q8_0:
        for j in range(8):
            b[:, 34 * j:34 * j + 2] = d
    else:
        b[:, 0:2] = d
        b[:, 2:4] = d
    m = pkg.QMatrix(dtype, n_in, n_out, b.reshape(-1))
    assert m.engine == "tcgen05"
    x = (rng.standard_normal((16, n_in)) * 0.1).astype(np.float32)
    first = m.matmul(x)
    for _ in range(40):
        assert m.matmul(x).tobytes() == first.tobytes()
    m.close()


def test_engines_by_dtype():
    for dtype, name in DTYPES:
        raw, _ = make_weight(dtype, 256, 128, 1)
        m = pkg.QMatrix(dtype, 256, 128, raw)
        assert m.engine == "tcgen05", name
        m.close()


def test_bad_shapes_are_refused():
    raw, _ = make_weight(orc.Q4_K, 256, 128, 1)
    with pytest.raises(pkg.DflError) as e:
        pkg.QMatrix(orc.Q4_K, 256, 128, raw[:-1])
    assert e.value.name == "BAD_SHAPE"
    m = pkg.QMatrix(orc.Q4_K, 256, 128, raw)
    with pytest.raises(pkg.DflError):
        m.matmul(np.zeros((17, 256), dtype=np.float32))
    m.close()


def test_argmax_top2_ties_signed_zero_nan_and_gap():
    rng = np.random.default_rng(4)
    v = 151936
    logits = rng.standard_normal((16, v)).astype(np.float32)
    logits[1, 5] = logits[1, 77777] = 9.0          # tie -> lowest index, gap 0
    logits[2, :] = -0.0
    logits[2, 100] = 0.0                            # +0 > -0 in total order
    logits[3, 151935] = 50.0                        # last element
    logits[4, 12345] = np.nan                       # NaN -> ~index
    am, gap = pkg.argmax_top2(logits)
    for r in range(16):
        want = orc.greedy_token(logits[r])
        if want < 0:
            assert am[r] == want
            continue
        assert am[r] == want
        row = logits[r].copy()
        top = row[want]
        row[want] = -np.inf
        assert gap[r] == np.float32(top) - np.float32(row.max())
    assert am[1] == 5 and gap[1] == 0.0
    assert am[2] == 100
    assert am[4] == ~12345


def test_config1_pipeline_matches_oracle_and_accepts_same_prefix():
    # the CPU-runnable verify / accept case at full size: 4096x4096 Q4_K, 4096 -> 32000 Q6_K head, 16 rows, greedy prefix acceptance
    h, v, n = 4096, 32000, 16
    raw1, _ = make_weight(orc.Q4_K, h, h, 101)
    raw2, _ = make_weight(orc.Q6_K, h, v, 102)
    rng = np.random.default_rng(103)
    x = rng.standard_normal((n, h)).astype(np.float32)
    hid = orc.matmul(orc.Q4_K, raw1, h, h, x)
    want = orc.matmul(orc.Q6_K, raw2, h, v, hid)
    want_arg = np.array([orc.greedy_token(want[r]) for r in range(n)], dtype=np.int32)
    w1 = pkg.QMatrix(orc.Q4_K, h, h, raw1)
    w2 = pkg.QMatrix(orc.Q6_K, h, v, raw2)
    pipe = pkg.C1Pipeline(w1, w2)
    # drafts: first 5 agree with the target, then seeded uniform ids
    draft = rng.integers(0, v, size=n).astype(np.int32)
    draft[:5] = want_arg[:5]
    am, gap, nacc, logits = pipe.step(x, draft, want_logits=True)
    np.testing.assert_allclose(logits, want, rtol=1e-2, atol=1e-3)
    assert np.array_equal(am, want_arg)
    want_acc = 0
    while want_acc < n and draft[want_acc] == want_arg[want_acc]:
        want_acc += 1
    assert nacc == want_acc
    s = np.sort(want, axis=1)
    np.testing.assert_allclose(gap, s[:, -1] - s[:, -2], rtol=0, atol=1e-4)
    pipe.close(); w1.close(); w2.close()
