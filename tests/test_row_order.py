"""Rows ordered ahead of the sampler (dfl_sampler_set_row_order): a registered order must change nothing the sampler
draws or decides, and an order that is not the row's own is ignored.  No GPU needed: the order is made with numpy."""
import numpy as np
import pytest

from dflb import pkg  # noqa: E402

NAN = float("nan")


def descending_key(rows):
    """The sampler's ordering key (crates/qwen-llm/src/sampling.rs:305-790: descending logit in the f32 total order)."""
    b = np.ascontiguousarray(rows, dtype=np.float32).view(np.uint32)
    asc = np.where(b & np.uint32(0x80000000), ~b, b | np.uint32(0x80000000))
    return ~asc


def row_order(rows):
    return np.ascontiguousarray(np.argsort(descending_key(rows), axis=1, kind="stable").astype(np.uint32))


def special_rows(rng, n, v):
    rows = (rng.standard_normal((n, v)) * 4).astype(np.float32)
    rows[0, rng.integers(0, v, 40)] = rows[0].max()              # ties at the top
    rows[1, rng.integers(0, v, 300)] = np.float32(-np.inf)       # masked tokens
    rows[2, ::7] = np.float32(0.0)
    rows[2, 3::7] = np.float32(-0.0)                             # +0 sorts before -0 in the total order
    rows[3] = np.round(rows[3])                                  # many ties everywhere
    if n > 4:
        rows[4, 17] = np.float32(np.inf)
    return rows


@pytest.mark.parametrize("cfg", [dict(temperature=0.7, top_p=0.95), dict(temperature=1.0), dict(temperature=0.8, top_k=50, min_p=0.02),
                                 dict(temperature=1.2, top_k=5000, top_p=0.9)])
def test_registered_order_keeps_the_sample_stream(cfg):
    rng = np.random.default_rng(3)
    n, v = 6, 5000
    rows = special_rows(rng, n, v)
    order = row_order(rows)
    plain, pre = pkg.Sampler(seed=11, **cfg), pkg.Sampler(seed=11, **cfg)
    pre.set_row_order(rows, order)
    for rep in range(3):
        for r in range(n):
            assert pre.sample(rows[r]) == plain.sample(rows[r].copy())
    assert pre.draws == plain.draws and pre.rng_state() == plain.rng_state()
    assert pre.preordered_rows == 3 * n and plain.preordered_rows == 0
    pre.set_row_order(None, None)
    assert pre.sample(rows[0]) == plain.sample(rows[0])
    assert pre.preordered_rows == 3 * n


def test_an_order_of_other_logits_is_ignored():
    rng = np.random.default_rng(4)
    n, v = 4, 4500
    rows = special_rows(rng, n, v)
    cfg = dict(temperature=0.9, top_p=0.9)
    plain = pkg.Sampler(seed=2, **cfg)
    want = [plain.sample(rows[r]) for r in range(n)]
    good = row_order(rows)
    bad = [good.copy() for _ in range(4)]
    bad[0][:, [10, 11]] = bad[0][:, [11, 10]]           # two neighbours swapped
    bad[1][:, 5] = bad[1][:, 6]                         # a repeated token
    bad[2][:, 100] = v + 3                              # a token outside the row
    bad[3][:] = np.arange(v, dtype=np.uint32)           # token order
    for o in bad:
        s = pkg.Sampler(seed=2, **cfg)
        s.set_row_order(rows, np.ascontiguousarray(o))
        assert [s.sample(rows[r]) for r in range(n)] == want
        assert s.rng_state() == plain.rng_state() and s.preordered_rows == 0
    # equal logits out of token order are not the sampler's order either
    tie = good.copy()
    top = np.flatnonzero(rows[0] == rows[0].max())
    assert top.size >= 2
    pos = [int(np.flatnonzero(tie[0] == t)[0]) for t in top[:2]]
    tie[0, pos] = tie[0, pos[::-1]]
    s = pkg.Sampler(seed=2, **cfg)
    s.set_row_order(rows, tie)
    assert [s.sample(rows[r]) for r in range(n)] == want
    assert s.preordered_rows == n - 1


def test_accept_prefix_over_registered_rows_and_nan_rows():
    rng = np.random.default_rng(5)
    n, v = 16, 4608
    for it in range(4):
        rows = (rng.standard_normal((n, v)) * 5).astype(np.float32)
        rows[:, :8] += 14.0
        rows[it, 20:40] = rows[it, :20]
        verified = [int(rng.integers(0, v))]
        for r in range(n - 1):
            verified.append(int(np.argmax(rows[r])) if rng.random() < 0.7 else int(rng.integers(0, v)))
        cfg = dict(temperature=0.7, top_p=0.95)
        sparse = None
        if it % 2:
            sparse = [(verified[r + 1], [(verified[r + 1], 0.75), ((verified[r + 1] + 1) % v, 0.25)]) for r in range(n - 1)]
        plain, pre = pkg.Sampler(seed=it, **cfg), pkg.Sampler(seed=it, **cfg)
        pre.set_row_order(rows, row_order(rows))
        a = pkg.accept_prefix(verified, rows, v, sparse, plain, 100, [])
        b = pkg.accept_prefix(verified, rows, v, sparse, pre, 100, [])
        assert a == b and plain.draws == pre.draws and plain.rng_state() == pre.rng_state()
        assert pre.preordered_rows >= a["retain_input_count"] and plain.preordered_rows == 0
    # the NaN of a reached row is still reported by its first token, generator untouched
    rows = np.zeros((3, v), dtype=np.float32)
    rows[:, 3] = 50.0
    rows[1, 777] = NAN
    rows[1, 4000] = NAN
    s = pkg.Sampler(temperature=1.0, seed=5)
    s.set_row_order(rows, row_order(np.nan_to_num(rows)))
    before = s.rng_state()
    with pytest.raises(pkg.DflError) as e:
        pkg.accept_prefix([0, 3, 3], rows, v, None, s, 100, [])
    assert "row 1" in str(e.value) and "token 777" in str(e.value) and s.rng_state() == before


def test_host_wait_policy_argument_check():
    for mode in ("block", "yield", "spin", "auto"):     # recorded; applied at a device's next use, so no GPU is touched
        pkg.set_host_wait(mode)
    with pytest.raises(pkg.DflError):
        pkg.check(pkg.lib().dfl_set_host_wait(7))


@pytest.mark.parametrize("workers", [1, 2, 5])
def test_worker_thread_limit_changes_nothing_that_is_decided(workers):
    rng = np.random.default_rng(8)
    n, v = 16, 4608
    rows = (rng.standard_normal((n, v)) * 5).astype(np.float32)
    rows[:, :8] += 14.0
    verified = [int(rng.integers(0, v))] + [int(np.argmax(rows[r])) if r % 5 else int(rng.integers(0, v)) for r in range(n - 1)]
    cfg = dict(temperature=0.7, top_p=0.95)
    plain, capped = pkg.Sampler(seed=3, **cfg), pkg.Sampler(seed=3, **cfg)
    capped.set_worker_threads(workers)
    for _ in range(3):
        a = pkg.accept_prefix(verified, rows, v, None, plain, 100, [])
        b = pkg.accept_prefix(verified, rows, v, None, capped, 100, [])
        assert a == b and plain.draws == capped.draws and plain.rng_state() == capped.rng_state()
