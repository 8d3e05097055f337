"""Generates tests/golden/*.npz from the CPU oracle (run in the build container: python tests/golden/make_golden.py).

The reference itself cannot run here (Rust + Metal), so the vectors come from the oracle restatement, which is pinned
to the reference's own known-answer tests in tests/test_oracle_*.py.  Fixtures are small and committed; the GPU tests
compare the CUDA path against them without needing anything but numpy.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import modelgen  # noqa: E402
import orc  # noqa: E402


def gemm_case():
    rng = np.random.default_rng(2024)
    out = {}
    for dtype, name in ((orc.Q4_K, "q4_k"), (orc.Q5_K, "q5_k"), (orc.Q6_K, "q6_k"), (orc.Q8_0, "q8_0"), (orc.BF16, "bf16")):
        n_in, n_out = 512, 136
        w = (rng.standard_normal((n_out, n_in)) * 0.02).astype(np.float32)
        raw = orc.quantize(dtype, w)
        x = rng.standard_normal((16, n_in)).astype(np.float32)
        out[f"{name}_raw"] = raw
        out[f"{name}_x"] = x
        out[f"{name}_deq_row0"] = orc.dequant(dtype, raw, n_in * n_out).reshape(n_out, n_in)[0]
        out[f"{name}_y"] = orc.matmul(dtype, raw, n_in, n_out, x)
    np.savez_compressed(os.path.join(HERE, "gemm_small.npz"), **out)


def verify_case():
    arch = modelgen.tiny_arch()
    T = modelgen.target_tensors(arch, seed=77)
    om = modelgen.OracleModel(arch, T)
    st = om.new_state(64, True)
    rng = np.random.default_rng(78)
    tokens = rng.integers(0, arch.vocab_size, size=20).astype(np.int32)
    logits, caps = [], []
    for i, t in enumerate(tokens):
        l, c = om.single_token(st, t, i, [1, 3])
        logits.append(l)
        caps.append(c)
    logits = np.stack(logits)
    ssm, conv = om.read_gdn(st, 1)
    np.savez_compressed(os.path.join(HERE, "verify_tiny.npz"), seed=77, tokens=tokens, logits=logits.astype(np.float32),
                        capture=np.stack(caps).astype(np.float32), argmax=np.array([orc.greedy_token(r) for r in logits], dtype=np.int32),
                        gdn1_ssm=ssm, gdn1_conv=conv)


if __name__ == "__main__":
    gemm_case()
    verify_case()
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))
