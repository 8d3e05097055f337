"""World-size-2 gloo test of the data-parallel host logic (sequence partition + counter gather)."""
import importlib
import os
import socket
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    dp = importlib.import_module("qwen-llm_b200.dp")
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    mine = dp.partition_sequences(7, world, rank)
    local = {"tokens": float(10 * len(mine)), "steps": float(len(mine)), "decode_ms": 100.0 + 50.0 * rank}
    total = dp.gather_counters(local)
    q.put((rank, mine, total))
    dist.barrier()
    dist.destroy_process_group()


def test_partition_is_a_disjoint_cover_and_seeds_do_not_depend_on_world():
    sys.path.insert(0, ROOT)
    dp = importlib.import_module("qwen-llm_b200.dp")
    for world in (1, 2, 4, 8):
        seen = sorted(i for r in range(world) for i in dp.partition_sequences(32, world, r))
        assert seen == list(range(32))
    assert dp.partition_sequences(3, 8, 5) == []
    assert len({dp.per_sequence_seed(7, i) for i in range(32)}) == 32
    with pytest.raises(ValueError):
        dp.partition_sequences(4, 2, 2)


def test_two_rank_gloo_gather():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res[0][1] == [0, 2, 4, 6] and res[1][1] == [1, 3, 5]
    for _, _, total in res:
        assert total == {"decode_ms": 150.0, "steps": 7.0, "tokens": 70.0}
