"""`bench.py --impl reference` on the host cores: the line the driver reads must carry the contract's keys and describe
the same workload as the main arm.  Runs the oracle port on a bounded sample (about twenty seconds here)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"],
                         cwd=ROOT, capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and "unavailable" not in d
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline",
                "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in d, key
    sys.path.insert(0, ROOT)
    import bench
    import bench_c2
    assert d["metric"] == bench.METRIC and d["unit"] == bench.UNIT
    assert d["value"] > 0 and d["higher_is_better"] is True and d["steps"] == 1
    assert set(d["config"]) >= {"workload"} and "model" not in d["config"]
    cb = d["cpu_baseline"]
    assert cb["kind"] in ("port", "reference") and cb["cores"] >= 1 and cb["sample"] and cb["value"] == d["value"]
    assert d["e2e"] == {"value": d["value"], "unit": d["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    # the same workload description as the main arm's line
    assert d["config"]["workload"] == bench_c2.WORKLOAD_C2
