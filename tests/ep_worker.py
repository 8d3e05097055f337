"""One rank of the expert-parallel parity check (launched by tests/test_moe_ep_gpu.py under torchrun).

Every rank builds the same seeded routed-expert model, rank r keeps experts [r*E/W, (r+1)*E/W); the packed verify of
the expert-parallel model must give every rank the same logits, and those must match a single-GPU model of all experts
(same arithmetic up to the order in which the experts' outputs are summed) and the CPU oracle.

Second phase (EP_WATCHDOG=1): between steps, with nothing in flight, rank 1 stops joining passes (it stays alive and
keeps its memory).  Rank 0's next pass then holds a collective nobody answers; its host watchdog must end it within
DFL_EP_TIMEOUT_MS by aborting the communicator, report COLLECTIVE, poison the session and refuse later passes."""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))


def main():
    import torch
    import torch.distributed as dist
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    import modelgen
    from dflb import pkg
    arch = modelgen.tiny_arch(expert_count=8, expert_used_count=2, expert_feed_forward_length=256, expert_shared_feed_forward_length=256)
    T = modelgen.target_tensors(arch, seed=11)
    idt = torch.zeros(128, dtype=torch.uint8, device=f"cuda:{local}")
    if rank == 0:
        idt.copy_(torch.frombuffer(bytearray(pkg.ep_unique_id()), dtype=torch.uint8))
    dist.broadcast(idt, 0)
    nccl_id = bytes(idt.cpu().numpy().tobytes())
    ep_model = pkg.Model(arch, T, device=local, ep=(rank, world, nccl_id))
    sess, scr = pkg.Session(ep_model, 64, False), pkg.Scratch(ep_model, 16, 1)
    rng = np.random.default_rng(5)
    rows = []
    start = 0
    for n in (16, 3, 1):
        tokens = rng.integers(0, arch.vocab_size, size=n)
        _, _, logits = pkg.packed_verify(ep_model, sess, scr, [arch.n_layer - 1], tokens, start, want_logits=True)
        rows.append(logits)
        start += n
    mine = torch.from_numpy(np.concatenate(rows)).to(f"cuda:{local}")
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine)
    ok = all(torch.equal(gathered[0], g) for g in gathered)            # every rank continues from identical values
    if rank == 0:
        full = pkg.Model(arch, T, device=local)
        s2, sc2 = pkg.Session(full, 64, False), pkg.Scratch(full, 16, 1)
        rng = np.random.default_rng(5)
        want = []
        start = 0
        for n in (16, 3, 1):
            tokens = rng.integers(0, arch.vocab_size, size=n)
            _, _, logits = pkg.packed_verify(full, s2, sc2, [arch.n_layer - 1], tokens, start, want_logits=True)
            want.append(logits)
            start += n
        want = np.concatenate(want)
        np.testing.assert_allclose(mine.cpu().numpy(), want, rtol=1e-4, atol=1e-5)
        assert ok, "ranks disagree"
        # ... and the CPU oracle (forward.rs:749-824 routing), at the tolerance of the single-GPU parity tests
        om = modelgen.OracleModel(arch, T)
        ost = om.new_state(64, False)
        rng = np.random.default_rng(5)
        pos = 0
        got = mine.cpu().numpy()
        for n in (16, 3, 1):
            tokens = rng.integers(0, arch.vocab_size, size=n)
            for i, t in enumerate(tokens):
                row, _ = om.single_token(ost, int(t), pos + i, [arch.n_layer - 1])
                np.testing.assert_allclose(got[pos + i], row, rtol=1e-2, atol=1e-3)
            pos += n
        print("EP_PARITY_OK", world, flush=True)
    dist.barrier()
    if os.environ.get("EP_WATCHDOG") == "1":
        torch.cuda.synchronize()
        dist.barrier()                      # between steps: nothing of either rank is in flight
        if rank == 0:
            import time
            tokens = np.arange(4) % arch.vocab_size
            t0 = time.monotonic()
            try:
                pkg.packed_verify(ep_model, sess, scr, [arch.n_layer - 1], tokens, start)
                outcome = "completed"
            except pkg.DflError as e:
                outcome = e.name
            dt = time.monotonic() - t0
            try:
                pkg.packed_verify(ep_model, sess, scr, [arch.n_layer - 1], tokens, start)
                later = "completed"
            except pkg.DflError as e:
                later = e.name
            sess2 = pkg.Session(ep_model, 64, False)
            try:
                pkg.packed_verify(ep_model, sess2, scr, [arch.n_layer - 1], tokens, 0)
                fresh = "completed"
            except pkg.DflError as e:
                fresh = e.name
            torch.cuda.synchronize()        # the context is still usable
            print("EP_WATCHDOG", outcome, later, fresh, f"{dt:.2f}", flush=True)
        # rank 1 joins no pass; it waits on the host for rank 0's result, then both leave without touching the
        # aborted communicator again
        store = dist.distributed_c10d._get_default_store()
        if rank == 0:
            store.set("ep_watchdog_done", "1")
        else:
            store.wait(["ep_watchdog_done"])
        sys.stdout.flush()
        os._exit(0)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
