"""The device-side row ordering for the host sampler: bit-exact against a stable numpy sort by the sampler's key
(crates/qwen-llm/src/sampling.rs:305-790), and invisible in what the sampled DFlash loop emits."""
import numpy as np
import pytest

import modelgen
from dflb import pkg
from test_row_order import row_order, special_rows

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,v", [(1, 1), (3, 31), (5, 2048), (5, 2049), (16, 4097), (16, 151936), (2, 300001)])
def test_sort_rows_equals_stable_numpy_sort(n, v):
    rng = np.random.default_rng(n * 1000003 + v)
    if v >= 2048 and n >= 5:
        rows = special_rows(rng, n, v)
    else:
        rows = (rng.standard_normal((n, v)) * 3).astype(np.float32)
    if v >= 31:
        rows[-1, 5] = np.float32(np.nan)                                    # positive NaN sorts first, negative NaN last
        rows[-1, 9] = np.frombuffer(np.uint32(0xFFC00001).tobytes(), dtype=np.float32)[0]
    got = pkg.sort_rows_desc(rows)
    assert got.dtype == np.uint32 and np.array_equal(got, row_order(rows))


def test_all_equal_and_two_valued_rows():
    v = 70000
    rows = np.zeros((3, v), dtype=np.float32)
    rows[1, ::2] = 1.0
    rows[2] = -0.0
    assert np.array_equal(pkg.sort_rows_desc(rows), row_order(rows))


@pytest.fixture(scope="module")
def world():
    arch = modelgen.tiny_arch()
    T = modelgen.target_tensors(arch, seed=3)
    cfg = modelgen.tiny_dflash_config(arch)
    D = modelgen.drafter_tensors(arch, cfg, seed=4)
    gm = pkg.Model(arch, T)
    gd = pkg.Drafter(gm, cfg, D)
    yield arch, gm, gd
    gd.close(); gm.close()


def test_verify_returns_the_order_of_its_own_logits(world):
    arch, gm, gd = world
    layer_ids = gd.layer_ids()
    sess, scr = pkg.Session(gm, 128), pkg.Scratch(gm, 16, len(layer_ids))
    rng = np.random.default_rng(2)
    for n in (16, 7):
        toks = rng.integers(0, arch.vocab_size, size=n)
        am, gap, logits, order = pkg.packed_verify(gm, sess, scr, layer_ids, toks, sess.kv_n_pos, want_logits=True, want_order=True)
        assert order.shape == logits.shape and np.array_equal(order, row_order(logits))
        assert np.array_equal(order[:, 0].astype(np.int32), am)
    # switched off again: a plain call still works and returns no order
    am, gap, logits = pkg.packed_verify(gm, sess, scr, layer_ids, rng.integers(0, arch.vocab_size, size=4), sess.kv_n_pos, want_logits=True)
    assert logits.shape == (4, arch.vocab_size)
    sess.close(); scr.close()


@pytest.mark.parametrize("kw", [dict(), dict(sparse_proposals=True)])
def test_sampled_loop_is_unchanged_by_device_row_order(world, kw):
    arch, gm, gd = world
    layer_ids = gd.layer_ids()
    prompt = np.random.default_rng(12).integers(0, arch.vocab_size, size=23)
    outs = []
    for dev in (False, True):
        s = pkg.Sampler(temperature=0.7, top_p=0.95, seed=1234)
        sess, scr, ds = pkg.Session(gm, 256), pkg.Scratch(gm, 16, len(layer_ids)), pkg.DSession(gd, 256)
        logits, _ = pkg.prefill(gm, sess, scr, layer_ids, prompt, 0, feed_drafter=ds)
        toks, stats = pkg.generate(gm, sess, scr, ds, s, logits, 48, device_row_order=dev, **kw)
        outs.append((toks.tolist(), stats.spec_steps, stats.accepted_drafts, s.draws, s.rng_state(), s.preordered_rows))
        # the registration ends with the call: a later row at the same address is sorted by the sampler itself
        before = s.preordered_rows
        s.sample(np.zeros(arch.vocab_size, dtype=np.float32))
        assert s.preordered_rows == before
        for x in (sess, scr, ds):
            x.close()
    assert outs[0][:5] == outs[1][:5]
    assert outs[0][5] == 0 and outs[1][5] >= outs[1][1]      # at least one row per step took the device's order
