"""Expert-parallel routed-expert verify on 2 GPUs of one box (skipped when fewer are visible)."""
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.gpu
def test_expert_parallel_verify_matches_single_gpu():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                        "--master-port", "29533", os.path.join(HERE, "ep_worker.py")], capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "EP_PARITY_OK 2" in r.stdout


@pytest.mark.gpu
def test_watchdog_ends_a_pass_whose_peer_does_not_join():
    # the peer stays alive and simply issues no pass (a host-made failure); plain peer transport, no multicast
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", EP_WATCHDOG="1", DFL_EP_TIMEOUT_MS="1500")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                        "--master-port", "29534", os.path.join(HERE, "ep_worker.py")], capture_output=True, text=True, timeout=600, env=env)
    assert "EP_PARITY_OK 2" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("EP_WATCHDOG")]
    assert line, r.stdout[-2000:] + r.stderr[-2000:]
    _, outcome, later, fresh, dt = line[0].split()
    assert outcome == "COLLECTIVE"                 # the watchdog gave up and aborted the communicator
    assert later == "POISONED"                     # the session of the failed pass is poisoned
    assert fresh == "COLLECTIVE"                   # and the model refuses passes on any session
    assert 1.4 <= float(dt) < 10.0
