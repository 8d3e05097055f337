#!/usr/bin/env python
"""Benchmark of the DFlash speculative-decoding step on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c1|c3|c5|c2v|c4v|c5v|gemm] [--impl reference]

Prints ONE JSON line on rank 0.  A "step" is one pass of the hot path over one batch of
seeded synthetic input:
  * workload c2 (default): one DFlash outer step (draft 16 -> packed verify -> greedy accept ->
    rollback) of the 9B-class hybrid Q4_K_M target with the 5-layer bf16 drafter, batch 1;
  * workload c1: the CPU-runnable verify/accept step (16x4096 . Q4_K 4096x4096, Q6_K head to
    32000, greedy prefix acceptance);
  * workload c3: the same target and drafter with sampled acceptance (T 0.7, top-p 0.95), 32 independent
    sequences split over the GPUs (strong scaling);
  * workload c5: the c2 loop after a long pre-filled context (--ctx, default 131072 positions, fp16 KV);
  * workloads c2v / c4v / c5v (packed verify only: dense, routed-expert, long context) and gemm are
    kernel-level side benches.
`value` is accepted tokens per second with inputs resident in HBM; `e2e` is the same metric
through the host-buffer C-ABI call (copies inside the timed region).  With N > 1 each rank
drives its own GPU on independent sequences (no collective on the data path): weak scaling.
`--impl reference` times the reference's CPU algorithm (the oracle port; the reference's own
Rust/llama.cpp build cannot be compiled in this image) on the host cores.
"""
import argparse
import ctypes as C
import importlib
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

METRIC = "accepted_tok_per_s"
UNIT = "tok/s"


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        try:
            rows = [r.split(",") for r in open(self.path).read().strip().splitlines() if r.strip()]
            sm = [float(r[1]) for r in rows]
            mx = [float(r[2]) for r in rows]
            reasons = set()
            for r in rows:
                for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7), ("sw_power_cap", 8)):
                    if r[col].strip().lower().startswith("active"):
                        reasons.add(name)
            if sm:
                top = sorted(sm)[len(sm) // 2:]  # samples under load: the upper half
                out = {"sm_mhz": statistics.median(top), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}
        except Exception:
            pass
        finally:
            try:
                os.unlink(self.path)
            except Exception:
                pass
        return out


# ---------------------------------------------------------------------------
# workload c1
# ---------------------------------------------------------------------------
C1_H, C1_V, C1_N = 4096, 32000, 16
C1_BYTES = C1_H * C1_H // 256 * 144 + C1_V * C1_H // 256 * 210  # 116,957,184 quantised weight bytes per step


def c1_inputs(seed, orc):
    rng = np.random.default_rng(seed)
    w1 = (rng.standard_normal((C1_H, C1_H)) * 0.02).astype(np.float32)
    w2 = (rng.standard_normal((C1_V, C1_H)) * 0.02).astype(np.float32)
    raw1, raw2 = orc.quantize(orc.Q4_K, w1), orc.quantize(orc.Q6_K, w2)
    x = rng.standard_normal((C1_N, C1_H)).astype(np.float32)
    return raw1, raw2, x, rng


def c1_cpu(orc, raw1, raw2, x, steps):
    """The reference's CPU algorithm for config 1: dequantise once (as a resident model would), then
    scalar f32 mat_vec rows, greedy argmax, prefix acceptance."""
    L = orc.lib()
    w1 = orc.dequant(orc.Q4_K, raw1, C1_H * C1_H)
    w2 = orc.dequant(orc.Q6_K, raw2, C1_H * C1_V)
    hid = np.zeros((C1_N, C1_H), dtype=np.float32)
    logits = np.zeros((C1_N, C1_V), dtype=np.float32)
    vp = lambda a: a.ctypes.data_as(C.c_void_p)
    t0 = time.perf_counter()
    arg = None
    for _ in range(steps):
        L.orc_matmul_f32(vp(w1), C.c_uint64(C1_H), C.c_uint64(C1_H), vp(x), C.c_int32(C1_N), vp(hid))
        L.orc_matmul_f32(vp(w2), C.c_uint64(C1_H), C.c_uint64(C1_V), vp(hid), C.c_int32(C1_N), vp(logits))
        arg = np.array([orc.greedy_token(logits[r]) for r in range(C1_N)], dtype=np.int32)
    dt = time.perf_counter() - t0
    return dt / steps, arg, int(L.orc_num_threads())


def run_gemm(args, device):
    """One weight matrix, 16 activation rows: the few-row GEMM alone against the HBM roofline.
    The pipeline object chains dtype[n_in -> n_out] with dtype[n_out -> n_in]; both launches are timed with
    CUDA events on the launching stream and replicas larger than L2 are cycled."""
    pkg = importlib.import_module("qwen-llm_b200")
    name, n_in, n_out = args.gemm.split(":")
    n_in, n_out = int(n_in), int(n_out)
    dt = {"q4_k": pkg.Q4_K, "q5_k": pkg.Q5_K, "q6_k": pkg.Q6_K, "q8_0": pkg.Q8_0, "bf16": pkg.BF16}[name]
    blk = {pkg.Q4_K: 144, pkg.Q5_K: 176, pkg.Q6_K: 210, pkg.Q8_0: 272, pkg.BF16: 512}[dt]
    rng = np.random.default_rng(7)

    def raw(k, n):
        nb = n * (k // 256)
        if dt == pkg.BF16:
            w = rng.standard_normal((n, k)).astype(np.float32) * 0.02
            return (w.view(np.uint32) >> 16).astype(np.uint16).view(np.uint8).reshape(-1)
        b = rng.integers(0, 256, size=(nb, blk), dtype=np.uint8)
        d = np.full(nb, 1e-4, dtype=np.float16).view(np.uint8).reshape(nb, 2)   # sane f16 block scales
        if dt == pkg.Q6_K:
            b[:, 208:210] = d
        elif dt == pkg.Q8_0:
            for j in range(8):
                b[:, 34 * j:34 * j + 2] = d
        else:
            b[:, 0:2] = d
            b[:, 2:4] = d
        return b.reshape(-1)

    bytes_one = (n_in // 256) * n_out * blk
    n_rep = max(2, int(300e6 // (2 * bytes_one)) + 1)
    pipes = []
    for _ in range(n_rep):
        a, b = pkg.QMatrix(dt, n_in, n_out, raw(n_in, n_out), device), pkg.QMatrix(dt, n_out, n_in, raw(n_out, n_in), device)
        pipes.append((a, b, pkg.C1Pipeline(a, b)))
    x = (rng.standard_normal((16, n_in)) * 0.1).astype(np.float32)
    for _, _, p in pipes:
        p.upload(x)
    for i in range(max(3, args.warmup)):
        pipes[i % n_rep][2].run_resident(16, 1)
    sampler = ClockSampler(device)
    sampler.start()
    pkg.gemm_timing_begin()
    for i in range(args.steps):
        pipes[i % n_rep][2].run_resident(16, 1)
    ms, n, nbytes = pkg.gemm_timing_end()
    clocks = sampler.stop()
    peak, kind = measured_peaks()
    gbs = nbytes / ms / 1e6
    return {"metric": "gemm_GBps", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": ms / args.steps, "higher_is_better": True, "dtype": name, "data": "synthetic",
            "config": {"workload": f"gemm: 16 rows x {name} {n_in}x{n_out} then {n_out}x{n_in}", "l2": f"{n_rep} replicas cycled, > 126 MB"},
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak, "traffic": None,
                         "peak_kind": kind, "launches_timed": n, "us_per_launch": ms / n * 1e3},
            "gpu_launches": n, "clocks": clocks}


def run_c1(args, rank, world, device):
    import orc
    pkg = importlib.import_module("qwen-llm_b200")
    import torch
    raw1, raw2, x, rng = c1_inputs(1234 + rank, orc)
    # replicas so that consecutive steps stream different HBM lines (weights < L2 otherwise)
    n_rep = 4
    reps = []
    for _ in range(n_rep):
        reps.append((pkg.QMatrix(pkg.Q4_K, C1_H, C1_H, raw1, device), pkg.QMatrix(pkg.Q6_K, C1_H, C1_V, raw2, device)))
    pipes = [pkg.C1Pipeline(a, b) for a, b in reps]
    am0, _, _, _ = pipes[0].step(x, np.zeros(C1_N, dtype=np.int32))
    emitted_per_step = 5  # drafts agree with the target on 4 rows -> 4 accepted + 1 correction
    draft = rng.integers(0, C1_V, size=C1_N).astype(np.int32)
    draft[:4] = am0[:4]
    if draft[4] == am0[4]:
        draft[4] = (draft[4] + 1) % C1_V
    for p in pipes:
        p.upload(x)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize(device)

    for i in range(args.warmup):
        pipes[i % n_rep].run_resident(C1_N, 1)
    launches0 = pkg.launch_count()
    sampler = ClockSampler(device)
    sampler.start()
    barrier()
    dev_ms = 0.0
    for i in range(args.steps):
        dev_ms += pipes[i % n_rep].run_resident(C1_N, 1)
    barrier()
    launches = pkg.launch_count() - launches0
    # end to end: host buffers in, host results out, every step
    for i in range(min(3, args.warmup)):
        pipes[i % n_rep].step(x, draft)
    barrier()
    t0 = time.perf_counter()
    nacc = 0
    for i in range(args.steps):
        _, _, a, _ = pipes[i % n_rep].step(x, draft)
        nacc += a
    barrier()
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop()
    assert nacc == 4 * args.steps, f"accepted prefix changed: {nacc}"
    t = torch.tensor([dev_ms, e2e_s * 1e3], dtype=torch.float64, device=f"cuda:{device}")
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    dev_ms, e2e_ms = float(t[0]), float(t[1])
    peak, peak_kind = measured_peaks()
    per_step_ms = dev_ms / args.steps
    achieved = C1_BYTES / (per_step_ms * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": emitted_per_step * args.steps * world / (dev_ms * 1e-3), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step_ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "u4/u6 weights, f32 accumulate", "data": "synthetic",
        "config": {"workload": "c1: 16x4096 . Q4_K 4096x4096 -> Q6_K 4096x32000 head, greedy prefix accept, 5 tok/step",
                   "l2": f"{n_rep} weight replicas cycled (468 MB > L2)", "parallelism": f"dp{world} independent sequences"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None, "peak_kind": peak_kind, "kernel": "few-row GEMM (gemm_ts_kernel Q4_K + Q6_K head; both GEMMs of the step)",
                     "algorithmic_bytes_per_step": C1_BYTES},
        "e2e": {"value": emitted_per_step * args.steps * world / (e2e_ms * 1e-3), "unit": UNIT,
                "h2d_bytes_per_step": int(x.nbytes + draft.nbytes), "d2h_bytes_per_step": int(C1_N * 8)},
        "gpu_launches": int(launches), "clocks": clocks,
    }
    if rank == 0 and world == 1:
        sec, arg, threads = c1_cpu(orc, raw1, raw2, x, 1)
        assert np.array_equal(arg, am0), "CPU oracle and GPU argmax differ"
        line["cpu_baseline"] = {"value": emitted_per_step / sec, "unit": UNIT, "cores": threads, "kind": "port",
                                "sample": "1 full config-1 step (weights dequantised once, outside the timed region)"}
    return line


def run_reference(args, rank, world):
    """Reference arm: the reference's CPU algorithm (oracle port) on the host cores."""
    if rank != 0:
        return None
    import orc
    if args.workload == "c1":
        raw1, raw2, x, _ = c1_inputs(1234, orc)
        for _ in range(min(args.warmup, 1)):
            c1_cpu(orc, raw1, raw2, x, 1)
        steps = max(1, min(args.steps, 5))
        sec, _, threads = c1_cpu(orc, raw1, raw2, x, steps)
        value = 5 / sec
        sample = f"{steps} full config-1 steps"
        workload = "c1"
    else:
        c2 = importlib.import_module("bench_c2")
        r = c2.reference_arm(args)
        return {"impl": "reference", "metric": METRIC, "value": r["value"], "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": r["block_s"] * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "f32", "data": "synthetic",
                "config": {"workload": c2.WORKLOAD_C2, "l2": "5.1 GB of weights per verify >> 126 MB L2",
                           "parallelism": f"dp{world}: one independent sequence per GPU, no collective"},
                "reference_step": "a step of this arm is one 16-row block through a 4-layer slice of the model (bounded sample); "
                                  "value = 4.4 emitted tokens / (layers' share x 32/4 + head share)",
                "extrapolated_full_step_ms": r["full_step_s"] * 1e3,
                "cpu_baseline": {"value": r["value"], "unit": UNIT, "cores": r["threads"], "kind": "port", "sample": r["sample"]},
                "e2e": {"value": r["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    return {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": {"workload": workload},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def with_secondary(line, args, rank, world, local):
    """On more than one GPU the same launch also measures the two partitions that are not plain replicas and appends them
    to the line as `secondary`: 32 sampled sequences split over the GPUs (strong scaling, end to end), and the packed
    verify of the routed-expert model with its experts split over the GPUs.  A watchdog prints the primary line and ends
    every rank if the extra measurements do not finish in time, so they can never cost the primary result."""
    import signal
    import copy

    def bail(signum, frame):
        if rank == 0:
            line["secondary"] = {"error": "secondary measurements did not finish within the time limit"}
            print(json.dumps(line), flush=True)
        os._exit(0)

    signal.signal(signal.SIGALRM, bail)
    signal.alarm(int(os.environ.get("DFL_BENCH_SECONDARY_LIMIT_S", "420")))
    c2 = importlib.import_module("bench_c2")
    sec = {}
    a3 = copy.copy(args)
    a3.workload, a3.steps, a3.warmup = "c3", 10, 3
    try:
        l3 = c2.run_c3(a3, rank, world, local)
        sec["c3_sampled_32_sequences"] = {"value": l3["value"], "unit": l3["unit"], "e2e": l3["e2e"]["value"], "scaling": l3.get("scaling"),
                                          "per_outer_step_ms": l3.get("per_outer_step_ms"), "workload": l3["config"]["workload"]}
    except Exception as e:
        sec["c3_sampled_32_sequences"] = {"error": f"{type(e).__name__}: {e}"}
    a4 = copy.copy(args)
    a4.workload, a4.steps, a4.warmup = "c4v", 10, 3
    try:
        l4 = c2.run_verify_only(a4, rank, world, local)
        sec["c4_routed_expert_verify"] = {"ms_per_verify": l4["value"], "parallelism": l4.get("parallelism"), "workload": l4["config"]["workload"]}
    except Exception as e:
        sec["c4_routed_expert_verify"] = {"error": f"{type(e).__name__}: {e}"}
    signal.alarm(0)
    line["secondary"] = sec
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default=os.environ.get("DFL_BENCH_WORKLOAD", "auto"))
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--gemm", default="q4_k:4096:24576", help="workload gemm only: dtype:n_in:n_out")
    ap.add_argument("--ctx", type=int, default=131072, help="workloads c5 / c5v: context length filled before timing")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.workload == "auto":
        args.workload = "c2" if os.path.exists(os.path.join(ROOT, "bench_c2.py")) else "c1"
    if args.impl == "reference":
        line = run_reference(args, rank, world)
        if line is not None:
            print(json.dumps(line), flush=True)
        return
    import torch
    if world > 1:
        torch.cuda.set_device(local)
        torch.distributed.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    if args.workload == "c1":
        line = run_c1(args, rank, world, local)
    elif args.workload == "gemm":
        line = run_gemm(args, local)
    elif args.workload in ("c2v", "c4v", "c5v"):
        line = importlib.import_module("bench_c2").run_verify_only(args, rank, world, local)
    elif args.workload == "c3":
        line = importlib.import_module("bench_c2").run_c3(args, rank, world, local)
    else:
        c2 = importlib.import_module("bench_c2")
        line = c2.run(args, rank, world, local)
        if world > 1 and args.workload == "c2" and os.environ.get("DFL_BENCH_SECONDARY", "1") != "0":
            line = with_secondary(line, args, rank, world, local)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
