"""The oracle's scalar primitives against the known answers the reference's own CPU tests hold for them
(crates/qwen-llm/src/forward.rs:1377-1414: primitives_smoke, gdn_output_scale_folds_into_rms_epsilon) and against an
independent numpy statement of the same formulas (forward.rs:1256-1309)."""
import ctypes as C

import numpy as np

import orc


def prim(kind, x, w=None, eps=0.0):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.zeros_like(x)
    wp = np.ascontiguousarray(w, dtype=np.float32) if w is not None else None
    p = lambda a: a.ctypes.data_as(C.c_void_p) if a is not None else None
    orc.check(orc.lib().orc_primitive(C.c_int32(kind), p(x), C.c_uint64(x.size), p(wp), C.c_float(eps), p(out)))
    return out


RMS, L2, SOFTMAX, SILU, SOFTPLUS, SIGMOID = range(6)


def test_primitives_smoke():
    # forward.rs:1376-1393
    a = prim(L2, [1.0, 2.0, 3.0], eps=1e-6)
    assert abs(np.sqrt((a * a).sum()) - 1.0) < 1e-3
    assert abs(prim(SILU, [1.0])[0] - 0.7310586) < 1e-5
    assert abs(prim(SOFTPLUS, [0.0])[0] - np.log(np.float32(2.0))) < 1e-5
    sm = prim(SOFTMAX, [1.0, 2.0, 3.0])
    assert abs(sm.sum() - 1.0) < 1e-5


def test_gdn_output_scale_folds_into_rms_epsilon():
    # forward.rs:1395-1414: rms_norm(x / sqrt(d), w, eps) == rms_norm(x, w, eps * d) within 2e-6
    d, eps = 128, np.float32(1e-6)
    scale = np.float32(1.0) / np.sqrt(np.float32(d))
    x = np.array([((i % 23) - 11.0) * 0.07 for i in range(d)], dtype=np.float32)
    w = np.array([0.5 + (i % 7) * 0.1 for i in range(d)], dtype=np.float32)
    old = prim(RMS, x * scale, w, eps)
    folded = prim(RMS, x, w, eps * d)
    assert np.abs(old - folded).max() < 2e-6


def test_primitives_equal_an_independent_statement():
    rng = np.random.default_rng(0)
    x = (rng.standard_normal(257) * 3).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(257)).astype(np.float32)
    f64 = x.astype(np.float64)
    np.testing.assert_allclose(prim(RMS, x, w, 1e-6), f64 / np.sqrt((f64 * f64).mean() + 1e-6) * w, rtol=2e-6)
    np.testing.assert_allclose(prim(L2, x, eps=1e-6), f64 / max(np.sqrt((f64 * f64).sum()), 1e-6), rtol=2e-6)
    e = np.exp(f64 - f64.max())
    np.testing.assert_allclose(prim(SOFTMAX, x), e / e.sum(), rtol=1e-5, atol=1e-9)
    np.testing.assert_allclose(prim(SILU, x), f64 / (1 + np.exp(-f64)), rtol=2e-6, atol=1e-7)
    np.testing.assert_allclose(prim(SIGMOID, x), 1 / (1 + np.exp(-f64)), rtol=2e-6)
    # softplus: identity above 20, exp below -20 (forward.rs:1287-1296)
    edge = np.array([-30.0, -20.5, -1.0, 0.0, 3.0, 20.5, 40.0], dtype=np.float32)
    want = np.where(edge > 20, edge, np.where(edge < -20, np.exp(edge.astype(np.float64)), np.log1p(np.exp(edge.astype(np.float64)))))
    np.testing.assert_allclose(prim(SOFTPLUS, edge), want, rtol=2e-6)
    # the max-form of the L2 norm keeps a zero vector at zero instead of dividing by zero (forward.rs:1269-1275)
    assert not np.isnan(prim(L2, np.zeros(8, dtype=np.float32), eps=1e-6)).any()
