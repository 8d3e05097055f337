"""Golden fixtures (tests/golden/*.npz, made by tests/golden/make_golden.py from the pinned oracle):
the oracle must keep reproducing them (CPU), and the CUDA path must match them (GPU)."""
import os

import numpy as np
import pytest

import modelgen
import orc

G = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
DT = {"q4_k": orc.Q4_K, "q5_k": orc.Q5_K, "q6_k": orc.Q6_K, "q8_0": orc.Q8_0, "bf16": orc.BF16}


def test_oracle_reproduces_gemm_fixture():
    z = np.load(os.path.join(G, "gemm_small.npz"))
    for name, dtype in DT.items():
        raw, x = z[f"{name}_raw"], z[f"{name}_x"]
        assert orc.dequant(dtype, raw, 512 * 136)[:512].tobytes() == z[f"{name}_deq_row0"].tobytes()
        assert orc.matmul(dtype, raw, 512, 136, x).tobytes() == z[f"{name}_y"].tobytes()


def test_oracle_reproduces_verify_fixture():
    z = np.load(os.path.join(G, "verify_tiny.npz"))
    arch = modelgen.tiny_arch()
    om = modelgen.OracleModel(arch, modelgen.target_tensors(arch, seed=int(z["seed"])))
    st = om.new_state(64, True)
    for i, t in enumerate(z["tokens"][:6]):
        l, c = om.single_token(st, t, i, [1, 3])
        np.testing.assert_allclose(l, z["logits"][i], rtol=1e-5, atol=1e-6)  # libm may differ across boxes by an ulp
        np.testing.assert_allclose(c, z["capture"][i], rtol=1e-5, atol=1e-6)


@pytest.mark.gpu
def test_cuda_gemm_matches_fixture():
    from dflb import pkg
    z = np.load(os.path.join(G, "gemm_small.npz"))
    for name, dtype in DT.items():
        m = pkg.QMatrix(dtype, 512, 136, z[f"{name}_raw"])
        assert m.dequant()[0].tobytes() == z[f"{name}_deq_row0"].tobytes()
        np.testing.assert_allclose(m.matmul(z[f"{name}_x"]), z[f"{name}_y"], rtol=1e-2, atol=1e-3)
        m.close()


@pytest.mark.gpu
def test_cuda_verify_matches_fixture():
    from dflb import pkg
    z = np.load(os.path.join(G, "verify_tiny.npz"))
    arch = modelgen.tiny_arch()
    gm = pkg.Model(arch, modelgen.target_tensors(arch, seed=int(z["seed"])))
    sess, scr = pkg.Session(gm, 64, True), pkg.Scratch(gm, 16, 2)
    tokens = z["tokens"]
    am1, _, l1 = pkg.packed_verify(gm, sess, scr, [1, 3], tokens[:16], 0, want_logits=True)
    cap1 = scr.read_capture(16)
    am2, _, l2 = pkg.packed_verify(gm, sess, scr, [1, 3], tokens[16:], 16, want_logits=True)
    logits = np.concatenate([l1, l2])
    np.testing.assert_allclose(logits, z["logits"], rtol=1e-2, atol=1e-3)
    np.testing.assert_allclose(cap1, z["capture"][:16], rtol=1e-2, atol=1e-3)
    s = np.sort(z["logits"], axis=1)
    safe = (s[:, -1] - s[:, -2]) > 1e-4
    assert np.array_equal(np.concatenate([am1, am2])[safe], z["argmax"][safe])
    ssm, conv = sess.read_gdn_state(1)
    np.testing.assert_allclose(ssm, z["gdn1_ssm"], rtol=1e-2, atol=1e-3)
    np.testing.assert_allclose(conv, z["gdn1_conv"], rtol=1e-2, atol=1e-3)
    for x in (sess, scr, gm):
        x.close()
