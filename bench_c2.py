"""Workload c2 of bench.py: greedy DFlash decode, 9B-class hybrid Q4_K_M target + 5-layer bf16 drafter,
batch 1, prompt 512 random ids, block 16.

One bench "step" is one DFlash outer step: draft 16 -> packed verify of 16 rows -> accept prefix ->
context append -> rollback.  Random-init weights make the drafter's own acceptance ~0, so acceptance
is controlled with the reference's replayed-draft mode (dflash_prefix_replay_drafts, qwen/dflash.rs:351-376):
drafts come from the true greedy continuation with seeded corruption, while the drafter still runs every
step so that no work is skipped.  The headline schedule accepts 3,3,4,3,4 drafts per step (mean emitted 4.4
tokens per step, the reference's measured acceptance, docs/PERF-LOG.md:22184-22187); the natural (alpha ~ 0) and
full-accept schedules are reported beside it.
"""
import ctypes as C
import importlib
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

PROMPT = 512
NEAR_TIE_MARGIN = 1e-4        # committed rows whose top-1 / top-2 gap is smaller are counted as near ties
PATTERN = [3, 3, 4, 3, 4]     # accepted drafts per step -> emitted 4,4,5,4,5 (mean 4.4)
KV_CAP = 4096


def _pkg():
    return importlib.import_module("qwen-llm_b200")


def _syn():
    return importlib.import_module("qwen-llm_b200.synthetic")


def schedule_history(cont, pattern, vocab):
    """Replay history that makes step k accept pattern[k % len] drafts: corrupt the draft after them."""
    hist = np.array(cont, dtype=np.int32).copy()
    e, k = 1, 0
    while True:
        a = pattern[k % len(pattern)]
        if e + a >= hist.size:
            break
        if a < 15:
            hist[e + a] = (hist[e + a] + 1) % vocab
        e += a + 1
        k += 1
    return hist


def tokens_for_steps(pattern, first_step, n_steps):
    return 1 + sum(pattern[(first_step + i) % len(pattern)] + 1 for i in range(n_steps))


class World:
    def __init__(self, device, seed, prompt_len=PROMPT, kv_cap=KV_CAP):
        pkg, syn = _pkg(), _syn()
        self.pkg = pkg
        self.kv_cap = kv_cap
        self.snapshot = None       # (blob, first logits) of the prefilled prompt: later fresh() calls restore it
        self.arch = syn.arch_9b()
        t0 = time.perf_counter()
        ents = syn.target_entries(self.arch, seed=seed, device=device)
        self.model = syn.build_model(self.arch, ents, device)
        self.sample_entries = None
        syn.free_entries(ents, device)
        self.cfg = syn.dflash_config_9b(self.arch)
        dents = syn.drafter_entries(self.arch, self.cfg, seed=seed + 1, device=device)
        self.drafter = syn.build_drafter(self.model, self.cfg, dents)
        syn.free_entries(dents, device)
        self.build_s = time.perf_counter() - t0
        self.layer_ids = self.drafter.layer_ids()
        self.prompt = np.random.default_rng(seed + 2).integers(0, self.arch.vocab_size, size=prompt_len).astype(np.int32)
        self.sess = self.scr = self.ds = None

    def fresh(self):
        pkg = self.pkg
        for x in (self.sess, self.scr, self.ds):
            if x is not None:
                x.close()
        self.sess = pkg.Session(self.model, self.kv_cap, True)
        self.scr = pkg.Scratch(self.model, 16, len(self.layer_ids))
        self.ds = pkg.DSession(self.drafter, self.kv_cap)
        if self.snapshot is not None:   # bitwise the state the prefill left (tests/test_snapshot_gpu.py)
            t0 = time.perf_counter()
            pkg.session_restore_snapshot(self.model, self.sess, self.ds, self.snapshot[0])
            self.restore_s = time.perf_counter() - t0
            return self.snapshot[1]
        t0 = time.perf_counter()
        logits, _ = pkg.prefill(self.model, self.sess, self.scr, self.layer_ids, self.prompt, 0, feed_drafter=self.ds)
        self.prefill_s = time.perf_counter() - t0
        self.snapshot = (pkg.session_snapshot(self.model, self.sess, self.ds), logits)
        self.restore_s = None
        return logits

    def gen(self, first_logits, max_tokens, **kw):
        return self.pkg.generate(self.model, self.sess, self.scr, self.ds, self.pkg.Sampler(), first_logits, max_tokens, **kw)


def one_hot(vocab, tok):
    l = np.full(vocab, -1.0, dtype=np.float32)
    l[tok] = 1.0
    return l


def run_schedule(w, cont, pattern, warm_steps, steps, runs_drafter=True):
    """Returns dict with device / wall timings of exactly `steps` outer steps after `warm_steps` warm-up steps."""
    V = w.arch.vocab_size
    hist = schedule_history(cont, pattern, V)
    logits = w.fresh()
    n_a = tokens_for_steps(pattern, 0, warm_steps)
    toks_a, _ = w.gen(logits, n_a, replay_history=hist, replay_runs_drafter=runs_drafter, replay_unchecked=True)
    assert np.array_equal(toks_a, cont[:n_a]), "warm-up output differs from the greedy continuation"
    n_b = tokens_for_steps(pattern, warm_steps, steps)
    launches0 = w.pkg.launch_count()
    t0 = time.perf_counter()
    toks_b, st = w.gen(one_hot(V, int(toks_a[-1])), n_b, replay_history=hist[n_a - 1:], replay_runs_drafter=runs_drafter,
                       replay_unchecked=True, verify_margin=NEAR_TIE_MARGIN)
    wall = time.perf_counter() - t0
    launches = w.pkg.launch_count() - launches0
    assert np.array_equal(toks_b, cont[n_a - 1:n_a - 1 + n_b]), "timed output differs from the greedy continuation"
    assert st.spec_steps == steps, (st.spec_steps, steps)
    emitted = n_b - 1
    dev_ms = st.draft_ms + st.verify_ms + st.restore_ms
    return {"emitted": emitted, "steps": steps, "dev_ms": dev_ms, "wall_ms": wall * 1e3, "draft_ms": st.draft_ms, "verify_ms": st.verify_ms,
            "restore_ms": st.restore_ms, "accept_ms": st.accept_ms, "append_ms": st.append_ms, "launches": launches,
            "restore_calls": st.restore_calls, "accepted": int(st.accepted_drafts), "committed_rows": int(st.committed_rows),
            "margin_rows": int(st.margin_rows)}


WORKLOAD_C2 = ("c2: 9B-class hybrid Q4_K_M target (32 layers, GDN:attn 3:1, H 4096, FFN 12288, V 151936) + 5-layer bf16 DFlash drafter, "
               "greedy, batch 1, prompt 512, block 16; replayed drafts accept 3,3,4,3,4 per step (4.4 emitted/step), drafter runs every step")


class CpuBlockSample:
    """The reference's CPU path on a bounded sample of the config-2 verify: one block = 16 consecutive single-token
    passes (forward.rs:173-220) through a 4-layer slice (3 GDN + 1 attention) with the real widths, plus the lm_head
    for every row.  `step()` runs and times one such block; `full_step_s(t)` scales a measured block time to the whole
    32-layer model: (layers part) x 32 / 4 + (head part)."""

    def __init__(self, arch, tensors):
        import modelgen
        import orc
        L = orc.lib()
        cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
        self.threads = int(L.orc_set_num_threads(int(cores)))   # all the cores this process may use, whatever OMP_NUM_THREADS says
        a4 = _pkg().Arch()
        for f, _ in arch._fields_:
            setattr(a4, f, getattr(arch, f))
        a4.n_layer = 4
        self.arch, self.n_layer_full = arch, arch.n_layer
        self.om = modelgen.OracleModel(a4, tensors)
        self.rng = np.random.default_rng(0)
        st = self.om.new_state(64, True)
        self.om.single_token(st, 1, 0, (), want_logits=True)          # dequantises every weight once (not timed)
        # the layers' share of a block, measured once: 16 passes without the head
        toks = self.rng.integers(0, arch.vocab_size, size=16)
        st = self.om.new_state(64, True)
        t0 = time.perf_counter()
        for i, t in enumerate(toks):
            self.om.single_token(st, t, i, (), want_logits=False)
        self.layers_s = time.perf_counter() - t0

    def step(self):
        toks = self.rng.integers(0, self.arch.vocab_size, size=16)
        st = self.om.new_state(64, True)
        t0 = time.perf_counter()
        for i, t in enumerate(toks):
            self.om.single_token(st, t, i, (), want_logits=True)
        return time.perf_counter() - t0

    def full_step_s(self, block_s):
        head_s = max(block_s - self.layers_s, 0.0)
        return self.layers_s * (self.n_layer_full / 4.0) + head_s

    def describe(self):
        return ("oracle port (the reference's scalar CPU algorithm, OpenMP over output rows): one block = 16 single-token passes through a "
                "4-layer (3 GDN + 1 attention) + lm_head slice with config-2 widths; tok/s scales the layers' share by 32/4; drafter not included")


def host_random_entries(arch, layers=(0, 1, 2, 3), seed=0):
    """Random valid quantised blocks generated on the host (fast): timing does not depend on the values."""
    import orc
    rng = np.random.default_rng(seed)
    H, F, V = arch.hidden_size, arch.intermediate_size, arch.vocab_size
    hd = arch.attn_head_dim
    q_dim, kv_dim = arch.n_q_heads * hd, arch.n_kv_heads * hd
    n_v, n_k = arch.gdn_n_v_heads, arch.gdn_n_k_heads
    conv_dim, v_dim = (2 * n_k + n_v) * 128, n_v * 128
    T = []
    blk_bytes = {orc.Q4_K: 144, orc.Q5_K: 176, orc.Q6_K: 210}

    def mat(name, dtype, n_in, n_out):
        nb = n_in * n_out // 256
        raw = rng.integers(0, 256, size=(nb, blk_bytes[dtype]), dtype=np.uint8)
        scale = np.frombuffer(np.float16(2e-4).tobytes(), dtype=np.uint8)
        if dtype == orc.Q6_K:
            raw[:, 208:210] = scale
        else:
            raw[:, 0:2] = scale
            raw[:, 2:4] = scale
        T.append((name, dtype, [n_in, n_out], raw.reshape(-1)))

    def vec(name, v, shape=None):
        a = np.ascontiguousarray(v, dtype=np.float32)
        T.append((name, orc.F32, shape or [a.size], a.view(np.uint8)))

    mat("token_embd.weight", orc.Q4_K, H, V)
    mat("output.weight", orc.Q6_K, H, V)
    vec("output_norm.weight", np.ones(H))
    for il in layers:
        b = f"blk.{il}."
        vec(b + "attn_norm.weight", np.ones(H))
        vec(b + "post_attention_norm.weight", np.ones(H))
        if il % 4 == 3:
            mat(b + "attn_q.weight", orc.Q4_K, H, 2 * q_dim)
            mat(b + "attn_k.weight", orc.Q4_K, H, kv_dim)
            mat(b + "attn_v.weight", orc.Q4_K, H, kv_dim)
            mat(b + "attn_output.weight", orc.Q4_K, q_dim, H)
            vec(b + "attn_q_norm.weight", np.ones(hd))
            vec(b + "attn_k_norm.weight", np.ones(hd))
        else:
            mat(b + "attn_qkv.weight", orc.Q6_K, H, conv_dim)
            mat(b + "attn_gate.weight", orc.Q4_K, H, v_dim)
            mat(b + "ssm_out.weight", orc.Q5_K, v_dim, H)
            vec(b + "ssm_alpha.weight", rng.standard_normal((n_v, H)) * 0.02, [H, n_v])
            vec(b + "ssm_beta.weight", rng.standard_normal((n_v, H)) * 0.02, [H, n_v])
            vec(b + "ssm_a", -rng.uniform(0.1, 2.0, n_v))
            vec(b + "ssm_dt.bias", rng.uniform(-1.0, 1.0, n_v))
            vec(b + "ssm_conv1d.weight", rng.standard_normal((conv_dim, 4)) * 0.3, [4, conv_dim])
            vec(b + "ssm_norm.weight", np.ones(128))
        mat(b + "ffn_gate.weight", orc.Q4_K, H, F)
        mat(b + "ffn_up.weight", orc.Q4_K, H, F)
        mat(b + "ffn_down.weight", orc.Q6_K, F, H)
    return T


def reference_arm(args):
    """bench.py --impl reference: the reference's CPU algorithm on the host cores.  One step = one 16-row block through
    the 4-layer slice (a bounded sample of the config-2 verify); ms_per_step is that measured time, `value` the
    accepted tokens per second of the full model it implies."""
    arch = _syn().arch_9b()
    sample = CpuBlockSample(arch, host_random_entries(arch))
    for _ in range(min(args.warmup, 2)):
        sample.step()
    steps = max(1, args.steps)
    times = [sample.step() for _ in range(steps)]
    block_s = sum(times) / steps
    emitted = sum(a + 1 for a in PATTERN) / len(PATTERN)
    full_s = sample.full_step_s(block_s)
    return {"value": emitted / full_s, "block_s": block_s, "full_step_s": full_s, "threads": sample.threads, "sample": sample.describe(),
            "layers_s": sample.layers_s}


def run(args, rank, world, device):
    import torch
    bench = importlib.import_module("bench")
    pkg = _pkg()
    long_ctx = int(args.ctx) if args.workload == "c5" else 0   # config 5: the same loop after a long pre-filled context
    w = World(device, seed=100 + rank, prompt_len=long_ctx, kv_cap=long_ctx + KV_CAP) if long_ctx else World(device, seed=100 + rank)
    V = w.arch.vocab_size
    steps, warm = args.steps, max(args.warmup, 3)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize(device)

    # pass 0: the true greedy continuation (also the natural, alpha ~ 0 schedule)
    need = tokens_for_steps([15], 0, warm + steps) + 16
    logits = w.fresh()
    t0 = time.perf_counter()
    n_nat = min(need, 1 + 2 * (warm + steps))
    cont_nat, st_nat = w.gen(logits, n_nat, verify_margin=NEAR_TIE_MARGIN)
    nat_wall = time.perf_counter() - t0
    # extend the continuation cheaply with full-accept replay of itself is impossible before it is known:
    # decode the rest with plain replay-free steps only as far as the schedules need
    cont = cont_nat
    if cont.size < need:
        logits = w.fresh()
        cont, _ = w.gen(logits, need, replay_history=cont_nat)   # replays what is known, then drafts naturally
    sampler = bench.ClockSampler(device)
    sampler.start()
    barrier()
    head = run_schedule(w, cont, PATTERN, warm, steps)
    barrier()
    clocks = sampler.stop()
    full = run_schedule(w, cont, [15], warm, steps)
    natural = {"emitted": int(st_nat.tokens_emitted) - 1, "steps": int(st_nat.spec_steps),
               "dev_ms": st_nat.draft_ms + st_nat.verify_ms + st_nat.restore_ms, "wall_ms": nat_wall * 1e3}
    # kernel-only timing of the dominant kernel on a few extra steps
    pkg.gemm_timing_begin()
    extra = run_schedule(w, cont, PATTERN, 1, 4)
    gemm_ms, gemm_n, gemm_bytes = pkg.gemm_timing_end()
    t = torch.tensor([head["dev_ms"], head["wall_ms"], full["dev_ms"], full["wall_ms"]], dtype=torch.float64, device=f"cuda:{device}")
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    dev_ms, wall_ms = float(t[0]), float(t[1])
    peak, peak_kind = bench.measured_peaks()
    vbytes = w.model.verify_weight_bytes()
    dbytes = w.drafter.weight_bytes()
    kv_bytes = 0
    if long_ctx:   # K and V rows one verify reads: attention layers x positions x 2 x n_kv x head_dim x 2 B (fp16)
        n_attn = sum(1 for il in range(w.arch.n_layer) if _syn().is_attn(w.arch, il))
        kv_bytes = n_attn * long_ctx * 2 * w.arch.n_kv_heads * w.arch.attn_head_dim * 2
    vbytes += kv_bytes
    rbytes = w.model.verify_resident_bytes() + kv_bytes   # what the step streams from HBM: Q6_K tiles hold a byte per code
    verify_ms = head["verify_ms"] / steps
    draft_ms = head["draft_ms"] / steps
    gemm_gbs = gemm_bytes / (gemm_ms * 1e-3) / 1e9 if gemm_ms > 0 else 0.0
    line = {
        "metric": bench.METRIC, "value": head["emitted"] * world / (dev_ms * 1e-3), "unit": bench.UNIT, "n_gpus": world, "steps": steps,
        "warmup": warm, "ms_per_step": dev_ms / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "u4/u5/u6 weights x f16 hi+lo activations, f32 accumulate; bf16 drafter", "data": "synthetic",
        "config": {"workload": (f"c5: the config-2 target and drafter after a context of {long_ctx} random ids pre-filled into an fp16 KV cache "
                                f"({kv_bytes / 2**30:.1f} GiB read per verify), greedy, batch 1, block 16; "
                                "replayed drafts accept 3,3,4,3,4 per step (4.4 emitted/step), drafter runs every step") if long_ctx else WORKLOAD_C2,
                   "l2": "5.1 GB of weights per verify >> 126 MB L2", "parallelism": f"dp{world}: one independent sequence per GPU, no collective"},
        # the unit of the roofline is one packed verify step: the quantised weight bytes it streams once (algorithmic bytes)
        # over its CUDA-event time, all kernels of the step included.  traffic: resident bytes x 1.04, the DRAM-bytes /
        # tile-bytes ratio an ncu capture of the dominant kernel showed on a smaller case (traffic grows with the bytes);
        # resident bytes exceed the algorithmic (ggml) bytes because Q6_K tiles hold one six-bit code per byte
        "roofline": {"bound": "hbm", "achieved": vbytes / (verify_ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": vbytes / (verify_ms * 1e-3) / 1e9 / peak, "traffic": 1.04 * rbytes, "resident_bytes": rbytes, "peak_kind": peak_kind,
                     "unit_of_work": "one packed verify step (16 rows through the 32-layer target and the lm_head), every kernel of the step",
                     "algorithmic_bytes": vbytes, "ms": verify_ms, "kernel": "gemm_ts_kernel<Q4_K | Q5_K | Q6_K> (the step's dominant kernel)",
                     "gemm_launches_only": {"GBps": gemm_gbs, "frac": gemm_gbs / peak, "launches_timed": gemm_n, "algorithmic_bytes_timed": gemm_bytes,
                                            "note": "every few-row GEMM launch of 4 extra outer steps (verify + draft) bracketed by CUDA events; "
                                                    "bracketing takes the launches out of their overlap, so the sum exceeds their share of a step"},
                     "draft_step": {"weight_bytes": dbytes, "ms": draft_ms, "GBps": dbytes / (draft_ms * 1e-3) / 1e9 if draft_ms > 0 else None}},
        "e2e": {"value": head["emitted"] * world / (wall_ms * 1e-3), "unit": bench.UNIT, "h2d_bytes_per_step": 2 * 16 * 4,
                "d2h_bytes_per_step": 3 * 16 * 4},
        "gpu_launches": int(head["launches"]), "clocks": clocks,
        # greedy continuation of the natural pass: committed verify rows and those whose top-1 / top-2 gap is below the margin
        # (a row this close to a tie may resolve differently under another f32 summation order)
        # committed rows of all three schedules (each row is one verify-pass logits row that decided an emitted token)
        "near_tie_rows": {"margin": NEAR_TIE_MARGIN,
                          "committed_rows": int(st_nat.committed_rows) + head["committed_rows"] + full["committed_rows"],
                          "rows_below_margin": int(st_nat.margin_rows) + head["margin_rows"] + full["margin_rows"]},
        "schedules": {
            "reference_like_4.4": {"tok_per_s": head["emitted"] / (head["dev_ms"] * 1e-3), "e2e_tok_per_s": head["emitted"] / (head["wall_ms"] * 1e-3),
                                   "ms_per_step": head["dev_ms"] / steps, "draft_ms": draft_ms, "verify_ms": verify_ms,
                                   "restore_ms": head["restore_ms"] / steps, "host_accept_ms": head["accept_ms"] / steps},
            "full_accept_16": {"tok_per_s": full["emitted"] / (full["dev_ms"] * 1e-3), "e2e_tok_per_s": full["emitted"] / (full["wall_ms"] * 1e-3),
                               "ms_per_step": full["dev_ms"] / steps},
            "natural_drafter": {"tok_per_s": natural["emitted"] / (natural["dev_ms"] * 1e-3) if natural["dev_ms"] else None,
                                "e2e_tok_per_s": natural["emitted"] / (natural["wall_ms"] * 1e-3), "steps": natural["steps"],
                                "mean_emitted": natural["emitted"] / max(natural["steps"], 1)}},
        "setup": {"build_s": w.build_s, "prefill_s": w.prefill_s, "snapshot_bytes": int(w.snapshot[0].size), "snapshot_restore_s": w.restore_s},
    }
    if rank == 0 and world == 1:
        try:
            syn = _syn()
            ents = syn.target_entries(w.arch, seed=100, device=device, layers=[0, 1, 2, 3])
            host = []
            for (name, dtype, shape, data, nb) in ents:
                raw = pkg.device_to_host(data, nb, device) if isinstance(data, int) else np.ascontiguousarray(data).view(np.uint8).reshape(-1)
                host.append((name, dtype, shape, raw))
            syn.free_entries(ents, device)
            sample = CpuBlockSample(w.arch, host)
            block_s = min(sample.step() for _ in range(2))
            per_verify = sample.full_step_s(block_s)
            emitted = sum(a + 1 for a in PATTERN) / len(PATTERN)
            line["cpu_baseline"] = {"value": emitted / per_verify, "unit": bench.UNIT, "cores": sample.threads, "kind": "port", "sample": sample.describe(),
                                    "cpu_block_s": block_s, "cpu_verify_s": per_verify}
        except Exception as e:  # the baseline is a reported extra; never lose the GPU line over it
            line["cpu_baseline"] = {"value": None, "unit": bench.UNIT, "cores": 0, "kind": "port", "sample": f"failed: {e}"}
    return line


def run_verify_only(args, rank, world, device):
    """Workloads c2v / c4v: packed verify steps only (16 rows, context 16..), for kernel profiling on the real shapes
    of config 2 (dense 9B-class hybrid) or config 4 (35B-A3B-shaped routed-expert hybrid, all experts on one GPU)."""
    bench = importlib.import_module("bench")
    pkg, syn = _pkg(), _syn()
    moe = args.workload == "c4v"
    arch = syn.arch_35b_a3b() if moe else syn.arch_9b()
    ents = syn.target_entries(arch, seed=100, device=device)
    ep = None
    if moe and world > 1:
        # expert parallel: every rank builds the same seeded tensors and keeps its own expert range
        import torch
        idt = torch.zeros(128, dtype=torch.uint8, device=f"cuda:{device}")
        if rank == 0:
            idt.copy_(torch.frombuffer(bytearray(pkg.ep_unique_id()), dtype=torch.uint8))
        torch.distributed.broadcast(idt, 0)
        ep = (rank, world, idt.cpu().numpy().tobytes())
    model = syn.build_model(arch, ents, device, ep)
    syn.free_entries(ents, device)
    ctx = int(getattr(args, "ctx", 0) or 0) if args.workload == "c5v" else 0
    sess, scr = pkg.Session(model, max(1024, ctx + 16 * (args.steps + args.warmup + 2)), True), pkg.Scratch(model, 16, 5)
    ids = [7, 15, 23, 31, 39] if moe else [5, 12, 18, 25, 31]
    rng = np.random.default_rng(0)
    pos = 0
    while pos < ctx:   # c5v: fill the fp16 KV cache (and the GDN state) with `ctx` random ids through the packed path
        pkg.packed_verify(model, sess, scr, ids, rng.integers(0, arch.vocab_size, size=16), pos)
        pos += 16
    for _ in range(max(args.warmup, 1)):
        pkg.packed_verify(model, sess, scr, ids, rng.integers(0, arch.vocab_size, size=16), pos)
        pos += 16
    launches0 = pkg.launch_count()
    pkg.gemm_timing_begin() if os.environ.get("DFL_GEMM_TIMING") else None
    t0 = time.perf_counter()
    for _ in range(args.steps):
        pkg.packed_verify(model, sess, scr, ids, rng.integers(0, arch.vocab_size, size=16), pos)
        pos += 16
    wall = (time.perf_counter() - t0) / args.steps
    if world > 1:
        import torch
        t = torch.tensor([wall], dtype=torch.float64, device=f"cuda:{device}")
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        wall = float(t[0])
    extra = {"parallelism": f"ep{world}: experts split over {world} GPUs, block outputs combined over peer memory (DFL_EP_COMBINE=nccl: ncclAllReduce)"} if ep else {}
    if os.environ.get("DFL_GEMM_TIMING"):
        ms, n, b = pkg.gemm_timing_end()
        extra = {"gemm_ms_per_step": ms / args.steps, "gemm_launches": n, "gemm_GBps": b / (ms * 1e-3) / 1e9}
    peak, kind = bench.measured_peaks()
    vb = model.verify_weight_bytes()
    if moe and not os.environ.get("DFL_MOE_ALL_EXPERTS"):
        # only the experts some row chose are streamed: expected count under the (near uniform) routing of random weights
        E, k = arch.expert_count, arch.expert_used_count
        frac = 1.0 - (1.0 - k / E) ** 16
        n_layer_local = arch.n_layer
        expert_bytes = n_layer_local * (E // world) * (2 * arch.hidden_size * arch.expert_feed_forward_length * 144 // 256 +
                                                       arch.hidden_size * arch.expert_feed_forward_length * 210 // 256)
        extra = {**extra, "model_weight_bytes": vb, "expected_active_expert_fraction": frac}
        vb = int(vb - expert_bytes * (1.0 - frac))
    if ctx:   # the KV bytes one verify reads: attention layers x positions x (K + V) x n_kv x head_dim x 2 B
        n_attn = sum(1 for il in range(arch.n_layer) if syn.is_attn(arch, il))
        kvb = n_attn * (ctx + 16 * args.warmup) * 2 * arch.n_kv_heads * arch.attn_head_dim * 2
        extra = {**extra, "kv_bytes_per_verify": kvb, "weight_bytes_per_verify": vb}
        vb += kvb
    return {"metric": "verify_ms", "value": wall * 1e3, "unit": "ms", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": wall * 1e3, "higher_is_better": False, "config": {"workload": (("c4v: packed verify only, 16 rows, 256 experts top-8 + shared, " + ("every expert streamed" if os.environ.get("DFL_MOE_ALL_EXPERTS") else "chosen experts streamed")) if moe
                                    else f"c5v: packed verify only, 16 rows over a context of {ctx} positions (fp16 KV)" if ctx
                                    else "c2v: packed verify only, 16 rows")},
            "roofline": {"bound": "hbm", "achieved": vb / wall / 1e9, "peak": peak, "unit": "GB/s", "frac": vb / wall / 1e9 / peak,
                         "traffic": None, "peak_kind": kind}, "gpu_launches": int(pkg.launch_count() - launches0), **extra}


# ---------------------------------------------------------------------------
# workload c3: sampled acceptance, 32 independent sequences, data parallel
# ---------------------------------------------------------------------------
C3_SEQS, C3_PROMPT, C3_T, C3_TOP_P, C3_SEED, C3_KV = 32, 1024, 0.7, 0.95, 0xC3, 2048
C3_THREADS = int(os.environ.get("DFL_C3_THREADS", "4"))   # host threads driving a rank's sequences in the end-to-end pass
# End-to-end pass on a host with few cores per driving thread (cores / (ranks x threads)).  Three switches, each "auto" by
# default and decided per launch from that ratio; the device-timed pass always runs the plain path:
#   DFL_C3_WAIT     block | spin   driving threads block instead of spinning while they wait for the GPU
#   DFL_C3_WORKERS  n              threads the sampler may use to build a block's rows ahead of its loop (1 = none)
#   DFL_C3_HOST_OFFLOAD  1 | 0     verify rows ordered on the device (the sampler then skips its sort, 45 % of its
#                                  work per row, for 0.5 ms of GPU time per step)
C3_WAIT = os.environ.get("DFL_C3_WAIT", "auto")
C3_WORKERS = os.environ.get("DFL_C3_WORKERS", "auto")
C3_HOST_OFFLOAD = os.environ.get("DFL_C3_HOST_OFFLOAD", "auto")


class Seq:
    """One independent sequence: its own target session, drafter session and request sampler."""

    def __init__(self, w, index):
        self.w, self.index = w, index
        self.prompt = np.random.default_rng(5000 + index).integers(0, w.arch.vocab_size, size=C3_PROMPT).astype(np.int32)
        self.seed = importlib.import_module("qwen-llm_b200.dp").per_sequence_seed(C3_SEED, index)   # independent of the rank count
        self.sess = self.ds = None

    def fresh(self):
        pkg, w = self.w.pkg, self.w
        self.close()
        self.sess = pkg.Session(w.model, C3_KV, True)
        self.ds = pkg.DSession(w.drafter, C3_KV)
        logits, _ = pkg.prefill(w.model, self.sess, w.scr, w.layer_ids, self.prompt, 0, feed_drafter=self.ds)
        return logits

    def sampler(self, at_draw=None):
        return self.w.pkg.Sampler(temperature=C3_T, top_p=C3_TOP_P, seed=self.seed, at_draw=at_draw)

    def gen(self, sampler, first_logits, max_tokens, **kw):
        return self.w.pkg.generate(self.w.model, self.sess, self.w.scr, self.ds, sampler, first_logits, max_tokens, **kw)

    def close(self):
        for x in (self.sess, self.ds):
            if x is not None:
                x.close()
        self.sess = self.ds = None


def forced(vocab, tok):
    """logits whose only sampled outcome is `tok` (the draw is still consumed)"""
    l = np.full(vocab, -np.inf, dtype=np.float32)
    l[tok] = 0.0
    return l


def run_c3(args, rank, world, device):
    """Sampled acceptance on the dense target and its drafter: sampled acceptance (temperature 0.7, top-p 0.95, fixed
    seeds, rejection sampling with one-hot coupling of the greedy drafts as the reference does for a drafter without
    selector, qwen/dflash.rs:508-522), 32 independent sequences with 1024-id prompts split round-robin over the GPUs.
    A step is one outer step of every sequence this rank owns.  Acceptance is controlled as in workload c2: the drafts
    replay the sequence's own sampled continuation (one-hot coupling keeps the serial sampler stream, so that
    continuation is exactly what plain sampled decoding emits) with seeded corruption, 3,3,4,3,4 accepted per step."""
    import torch
    bench = importlib.import_module("bench")
    w = World(device, seed=100, prompt_len=16)   # the same weights on every rank: data parallel replicas
    pkg = w.pkg
    V = w.arch.vocab_size
    steps, warm = args.steps, max(args.warmup, 3)
    w.scr = pkg.Scratch(w.model, 16, len(w.layer_ids))
    dp = importlib.import_module("qwen-llm_b200.dp")
    seqs = [Seq(w, i) for i in dp.partition_sequences(C3_SEQS, world, rank)]

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize(device)

    # pass 0 per sequence: the sampled continuation itself (natural drafter, acceptance ~ 0 with random weights)
    need = tokens_for_steps(PATTERN, 0, warm + 2 * steps) + 16   # warm-up, the device-timed pass, the end-to-end pass
    nat = {"emitted": 0, "steps": 0, "dev_ms": 0.0, "wall_ms": 0.0}
    state = []
    t_setup = time.perf_counter()
    for q in seqs:
        logits = q.fresh()
        t0 = time.perf_counter()
        cont, st = q.gen(q.sampler(), logits, need)
        nat["wall_ms"] += (time.perf_counter() - t0) * 1e3
        nat["emitted"] += int(st.tokens_emitted) - 1
        nat["steps"] += int(st.spec_steps)
        nat["dev_ms"] += st.draft_ms + st.verify_ms + st.restore_ms
        hist = schedule_history(cont, PATTERN, V)
        logits = q.fresh()
        n_a = tokens_for_steps(PATTERN, 0, warm)
        toks_a, _ = q.gen(q.sampler(), logits, n_a, replay_history=hist, replay_runs_drafter=True, replay_unchecked=True)
        assert np.array_equal(toks_a, cont[:n_a]), "warm-up output differs from the plain sampled continuation"
        state.append((cont, hist, n_a, int(toks_a[-1])))
    setup_s = time.perf_counter() - t_setup
    n_b = tokens_for_steps(PATTERN, warm, steps)
    clock = bench.ClockSampler(device)
    clock.start()
    barrier()
    launches0 = pkg.launch_count()
    tot = {"emitted": 0, "dev_ms": 0.0, "draft_ms": 0.0, "verify_ms": 0.0, "restore_ms": 0.0, "accept_ms": 0.0}
    t0 = time.perf_counter()
    for q, (cont, hist, n_a, last) in zip(seqs, state):
        toks_b, st = q.gen(q.sampler(at_draw=n_a - 1), forced(V, last), n_b, replay_history=hist[n_a - 1:], replay_runs_drafter=True,
                           replay_unchecked=True)
        assert np.array_equal(toks_b, cont[n_a - 1:n_a - 1 + n_b]), "timed output differs from the plain sampled continuation"
        assert st.spec_steps == steps, (st.spec_steps, steps)
        tot["emitted"] += n_b - 1
        for k in ("draft_ms", "verify_ms", "restore_ms", "accept_ms"):
            tot[k] += getattr(st, k)
    torch.cuda.synchronize(device)
    wall_serial_ms = (time.perf_counter() - t0) * 1e3
    launches = pkg.launch_count() - launches0
    barrier()
    clocks = clock.stop()
    # End-to-end pass: the same number of further steps of every sequence, driven by C3_THREADS host threads, each with
    # its own scratch and its own share of the sequences (a session is only ever touched by one thread).  While one
    # thread's sequence is in the host sampler another thread's sequence keeps the GPU busy.
    import threading
    n_done = n_b - 1           # tokens emitted by the device-timed pass, after the n_a of the warm-up
    n_c = tokens_for_steps(PATTERN, warm + steps, steps)
    threads = max(1, min(C3_THREADS, len(seqs)))
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    per_driver = cores / float(world * threads)          # host cores per driving thread
    scarce = per_driver <= 2.0    # measured: device row order gains 8 % at one core per driving thread, 7 % at two, loses at eight
    offload = C3_HOST_OFFLOAD == "1" or (C3_HOST_OFFLOAD == "auto" and scarce)
    workers = int(C3_WORKERS) if C3_WORKERS != "auto" else (0 if per_driver >= 6 else max(1, int(per_driver)))
    # spinning waits are the faster ones as long as every thread has a core of its own
    block = C3_WAIT == "block" or (C3_WAIT == "auto" and world * threads * (workers or 6) > cores)
    if block:
        pkg.set_host_wait("block")
    scratches = [w.scr] + [pkg.Scratch(w.model, 16, len(w.layer_ids)) for _ in range(threads - 1)]
    errors, emitted_e2e = [], [0] * threads

    def drive(ti):
        try:
            for q, (cont, hist, n_a, last) in list(zip(seqs, state))[ti::threads]:
                at = n_a - 1 + n_done
                smp = q.sampler(at_draw=at)
                smp.set_worker_threads(workers)
                toks_c, st = pkg.generate(w.model, q.sess, scratches[ti], q.ds, smp, forced(V, int(cont[at])), n_c,
                                          replay_history=hist[at:], replay_runs_drafter=True, replay_unchecked=True,
                                          device_row_order=offload)
                assert np.array_equal(toks_c, cont[at:at + n_c]), "end-to-end output differs from the plain sampled continuation"
                assert st.spec_steps == steps, (st.spec_steps, steps)
                emitted_e2e[ti] += n_c - 1
        except Exception as e:   # surfaced after the join
            errors.append(e)

    barrier()
    t0 = time.perf_counter()
    pool = [threading.Thread(target=drive, args=(ti,)) for ti in range(threads)]
    for t in pool:
        t.start()
    for t in pool:
        t.join()
    torch.cuda.synchronize(device)
    wall_ms = (time.perf_counter() - t0) * 1e3
    if block:
        pkg.set_host_wait("auto")
    if errors:
        raise errors[0]
    for sc in scratches[1:]:
        sc.close()
    tot["dev_ms"] = tot["draft_ms"] + tot["verify_ms"] + tot["restore_ms"]
    # whole-job counters: times take the max over ranks, emitted tokens the sum
    g = dp.gather_counters({"dev_ms": tot["dev_ms"], "wall_ms": wall_ms, "emitted": float(tot["emitted"]), "emitted_e2e": float(sum(emitted_e2e))},
                           device=f"cuda:{device}")
    dev_ms, wall_max, emitted, emitted_wall = g["dev_ms"], g["wall_ms"], g["emitted"], g["emitted_e2e"]
    peak, peak_kind = bench.measured_peaks()
    vbytes = w.model.verify_weight_bytes()
    n_steps_rank = steps * len(seqs)
    verify_ms = tot["verify_ms"] / n_steps_rank
    gbs = vbytes / (verify_ms * 1e-3) / 1e9
    for q in seqs:
        q.close()
    return {
        "metric": bench.METRIC, "value": emitted / (dev_ms * 1e-3), "unit": bench.UNIT, "n_gpus": world, "steps": steps, "warmup": warm,
        "ms_per_step": dev_ms / steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "u4/u5/u6 weights x f16 hi+lo activations, f32 accumulate; bf16 drafter; f64 host sampler", "data": "synthetic",
        "config": {"workload": f"c3: config-2 target + drafter, sampled acceptance T={C3_T} top-p={C3_TOP_P}, fixed seeds, one-hot rejection coupling; "
                               f"{C3_SEQS} independent sequences, prompt {C3_PROMPT}, block 16; replayed drafts accept 3,3,4,3,4 per step; "
                               "a step = one outer step of every sequence of the rank",
                   "l2": "5.1 GB of weights per verify >> 126 MB L2",
                   "parallelism": f"dp{world}: {C3_SEQS} sequences round-robin over {world} GPU(s), full replica each, no collective in the loop"},
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak, "traffic": None, "peak_kind": peak_kind,
                     "kernel": "one packed verify (all kernels), weight bytes / CUDA-event time"},
        "e2e": {"value": emitted_wall / (wall_max * 1e-3), "unit": bench.UNIT, "h2d_bytes_per_step": len(seqs) * 2 * 16 * 4,
                "d2h_bytes_per_step": len(seqs) * (16 * V * 4 * (2 if offload else 1) + 3 * 16 * 4),
                "host_policy": {"cores_per_driving_thread": per_driver, "wait": "block" if block else "spin",
                                "sampler_worker_threads": workers or "host concurrency", "row_order": "device" if offload else "host"}, "host_threads": threads,
                "one_thread_tok_per_s": tot["emitted"] / (wall_serial_ms * 1e-3)},
        "gpu_launches": int(launches), "clocks": clocks,
        "per_outer_step_ms": {"draft": tot["draft_ms"] / n_steps_rank, "verify": verify_ms, "restore": tot["restore_ms"] / n_steps_rank,
                              "host_accept": tot["accept_ms"] / n_steps_rank, "wall_one_thread": wall_serial_ms / n_steps_rank,
                              "wall_threads": wall_ms / n_steps_rank},
        "natural_drafter": {"tok_per_s": nat["emitted"] / (nat["dev_ms"] * 1e-3) if nat["dev_ms"] else None,
                            "e2e_tok_per_s": nat["emitted"] / (nat["wall_ms"] * 1e-3), "mean_emitted": nat["emitted"] / max(nat["steps"], 1)},
        "setup": {"build_s": w.build_s, "sequences_on_rank0": len(seqs), "prefill_and_continuation_s": setup_s},
    }
