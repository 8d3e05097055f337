"""CPU restatement of the DFlash 2 path selector (test infrastructure: only tests, the smoke check and the bench's CPU
baseline may import this).

Follows crates/qwen-llm/src/metal_dflash.rs: DFlash2Codebook (:3163-3340), select_draft_path (:17176-17251), the walk of
draft_block_sampled (:17349-17409) and diagnose_dflash2_selector_walk (:3472-3620); the top-16 rule is
kernel_topk16_f32 / topk16_better / f32_total_order_key (kernels/dflash2.metal:69-170).  Pinned by the reference's own
selector tests (metal_dflash/tests.rs:2862-3055), restated in tests/test_selector.py.
"""
import math
import struct

import numpy as np

F32, F16, Q8_0, Q4_K, BF16 = 0, 1, 8, 12, 30
TOP_K = 16


def total_order_key(v):
    """f32_total_order_key: signed 32-bit key whose integer order is the IEEE total order."""
    bits = np.asarray(v, dtype=np.float32).view(np.int32).astype(np.int64)
    return np.where(bits < 0, bits ^ 0x7FFFFFFF, bits)


def topk16(x):
    """ids, vals [rows][16]: descending by total-order key, ties to the lower index; slots beyond the row length (and
    slots an element worse than (-inf, 0xFFFFFFFF) would take) keep the sentinel (id -1, -inf)."""
    x = np.asarray(x, dtype=np.float32)
    rows, n = x.shape
    ids = np.full((rows, TOP_K), -1, dtype=np.int32)
    vals = np.full((rows, TOP_K), -np.inf, dtype=np.float32)
    sentinel_key = int(total_order_key(np.float32(-np.inf)))
    for r in range(rows):
        key = total_order_key(x[r])
        order = np.lexsort((np.arange(n), -key))[:TOP_K]
        j = 0
        for i in order:
            if key[i] < sentinel_key:   # never displaces the initial (-inf, 0xFFFFFFFF) entry
                break
            ids[r, j] = i
            vals[r, j] = x[r, i]
            j += 1
    return ids, vals


def _f16(bits):
    return np.array([bits], dtype=np.uint16).view(np.float16).astype(np.float32)[0]


class Codebook:
    """DFlash2Codebook: [rank, n_rows] in ggml storage, one rank-wide row per token id."""

    def __init__(self, dtype, rank, n_rows, raw):
        raw = bytes(raw)
        if rank == 0 or n_rows == 0:
            raise ValueError("selector codebook dimensions must be nonzero")
        layout = {Q4_K: (256, 144), Q8_0: (32, 34), F32: (1, 4), F16: (1, 2), BF16: (1, 2)}
        if dtype not in layout:
            raise ValueError("selector codebook dtype must be Q4_K/Q8_0/F32/F16/BF16")
        el, nb = layout[dtype]
        if rank % el:
            raise ValueError("selector codebook rank is not block-aligned")
        if dtype == Q4_K and rank != 256:
            raise ValueError("Q4_K selector codebook rank must be 256")
        self.row_bytes = rank // el * nb
        if len(raw) != self.row_bytes * n_rows:
            raise ValueError("selector codebook payload size mismatch")
        self.dtype, self.rank, self.n_rows, self.raw = dtype, rank, n_rows, raw

    def dequant_row(self, row):
        if row < 0 or row >= self.n_rows:
            raise IndexError("selector codebook row out of range")
        p = self.raw[row * self.row_bytes:(row + 1) * self.row_bytes]
        if self.dtype == F32:
            return np.frombuffer(p, dtype=np.float32).copy()
        if self.dtype == F16:
            return np.frombuffer(p, dtype=np.float16).astype(np.float32)
        if self.dtype == BF16:
            return (np.frombuffer(p, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)
        if self.dtype == Q8_0:
            out = np.zeros(self.rank, dtype=np.float32)
            for b in range(self.rank // 32):
                blk = p[34 * b:34 * b + 34]
                d = _f16(struct.unpack("<H", blk[:2])[0])
                out[32 * b:32 * b + 32] = d * np.frombuffer(blk[2:], dtype=np.int8).astype(np.float32)
            return out
        # Q4_K, one super-block: value = d * sc * q - dmin * m, each product rounded to f32 (ggml's order)
        d, dmin = _f16(struct.unpack("<H", p[0:2])[0]), _f16(struct.unpack("<H", p[2:4])[0])
        sc, q = p[4:16], np.frombuffer(p[16:144], dtype=np.uint8)
        out = np.zeros(256, dtype=np.float32)

        def scale_min(j):
            if j < 4:
                return sc[j] & 63, sc[j + 4] & 63
            return (sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4), (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4)

        for j in range(4):
            s1, m1 = scale_min(2 * j)
            s2, m2 = scale_min(2 * j + 1)
            d1, mm1 = np.float32(d * np.float32(s1)), np.float32(dmin * np.float32(m1))
            d2, mm2 = np.float32(d * np.float32(s2)), np.float32(dmin * np.float32(m2))
            ql = q[32 * j:32 * j + 32]
            out[64 * j:64 * j + 32] = d1 * (ql & 0xF).astype(np.float32) - mm1
            out[64 * j + 32:64 * j + 64] = d2 * (ql >> 4).astype(np.float32) - mm2
        return out


def _scores(pred_row, succ, hrow, cand_ids, unary):
    """per candidate: unary + sum_r (pred[r] * h[r]) * succ[r], accumulated in f32 in index order; None for sentinels"""
    gate = (pred_row * hrow).astype(np.float32)
    out = []
    for b, cand in enumerate(cand_ids):
        cand = int(cand)
        if cand < 0 or cand >= succ.n_rows:
            out.append(None)
            continue
        srow = succ.dequant_row(cand)
        dot = np.float32(0.0)
        for r in range(len(gate)):
            dot = np.float32(dot + np.float32(gate[r] * srow[r]))
        out.append(np.float32(np.float32(unary[b]) + dot))
    return out


def walk_greedy(pred, succ, top_k, rank, carry, n, ids, vals, sel_h):
    """select_draft_path: (tokens[n], per-depth list of candidate scores (None = not scored), per-depth chosen index)."""
    ids = np.asarray(ids, dtype=np.int32).reshape(n, top_k)
    vals = np.asarray(vals, dtype=np.float32).reshape(n, top_k)
    sel_h = np.asarray(sel_h, dtype=np.float32).reshape(n, rank)
    tokens = [int(ids[0, 0])] * n
    depth_scores, depth_choice = [], []
    pred_row = pred.dequant_row(int(carry))
    for pos in range(1, n):
        scores = _scores(pred_row, succ, sel_h[pos], ids[pos], vals[pos])
        best_b, best = 0, np.float32(-np.inf)
        for b, sc in enumerate(scores):
            if sc is not None and sc > best:   # strict: the first candidate wins ties, NaN never wins
                best, best_b = sc, b
        depth_scores.append(scores)
        depth_choice.append(best_b)
        chosen = int(ids[pos, best_b])
        tokens[pos] = chosen
        pred_row = pred.dequant_row(chosen)
    return tokens, depth_scores, depth_choice


def walk_sampled(pred, succ, top_k, rank, carry, n, ids, vals, sel_h, proposal_sampler):
    """draft_block_sampled's walk: (tokens[n], [(token, [(cand, weight), ...]) per draft position])."""
    cfg = proposal_sampler.config
    if cfg.temperature <= 0.0 or cfg.top_k != 0 or cfg.top_p != 1.0 or cfg.min_p != 0.0:
        raise ValueError("DFlash 2 proposal sampler must use temperature without target filters")
    ids = np.asarray(ids, dtype=np.int32).reshape(n, top_k)
    vals = np.asarray(vals, dtype=np.float32).reshape(n, top_k)
    sel_h = np.asarray(sel_h, dtype=np.float32).reshape(n, rank)
    tokens = [int(ids[0, 0])] * n
    proposals = []
    pred_row = pred.dequant_row(int(carry))
    for pos in range(1, n):
        scores = [(-math.inf if sc is None else float(sc)) for sc in _scores(pred_row, succ, sel_h[pos], ids[pos], vals[pos])]
        dist = proposal_sampler.sample_with_distribution(scores)
        token = int(ids[pos, dist.token])
        if token < 0 or token >= pred.n_rows:
            raise ValueError("sampled selector returned an invalid token")
        proposals.append((token, [(int(ids[pos, c]), w) for c, w in dist.candidates if w > 0.0]))
        tokens[pos] = token
        pred_row = pred.dequant_row(token)
    return tokens, proposals
