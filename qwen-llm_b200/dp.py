"""Data-parallel plumbing for independent sequences: one process per GPU, no collective on the data path.

A sequence's state (KV, GDN state, drafter context, sampler) never interacts with another's
(crates/qwen-llm/src/metal_forward/mod.rs:2092-2158; sampling.rs:1-7), so sequences are dealt round-robin to
ranks and only counters are gathered at the end (one all_reduce of a few scalars, MAX for times, SUM for tokens).
"""
from typing import Dict, List


def partition_sequences(n_sequences: int, world: int, rank: int) -> List[int]:
    """Indices of the sequences rank `rank` owns (round-robin)."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError("bad world/rank")
    return list(range(rank, n_sequences, world))


def per_sequence_seed(base_seed: int, sequence_index: int) -> int:
    """Seed of sequence i: independent of how sequences are spread over ranks, so results do not depend on N."""
    return (base_seed * 0x9E3779B97F4A7C15 + sequence_index * 0xBF58476D1CE4E5B9) & ((1 << 64) - 1)


def gather_counters(local: Dict[str, float], device=None, group=None) -> Dict[str, float]:
    """Whole-job counters: keys ending in `_ms` / `_s` take the MAX over ranks (the job ends with its slowest rank),
    every other key is SUMmed.  Works on any torch.distributed backend (NCCL on GPUs, gloo on CPU)."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return dict(local)
    keys = sorted(local)
    t_max = torch.tensor([local[k] for k in keys if k.endswith(("_ms", "_s"))], dtype=torch.float64, device=device)
    t_sum = torch.tensor([local[k] for k in keys if not k.endswith(("_ms", "_s"))], dtype=torch.float64, device=device)
    if t_max.numel():
        dist.all_reduce(t_max, op=dist.ReduceOp.MAX, group=group)
    if t_sum.numel():
        dist.all_reduce(t_sum, op=dist.ReduceOp.SUM, group=group)
    out, im, isum = {}, 0, 0
    for k in keys:
        if k.endswith(("_ms", "_s")):
            out[k] = float(t_max[im]); im += 1
        else:
            out[k] = float(t_sum[isum]); isum += 1
    return out
