"""The in-kernel record exchange across real GPUs (needs at least two; skipped otherwise): ranks are
child processes, one per GPU, launched with torch.distributed.run on 127.0.0.1.  Covers the fused
single-launch path over CUDA IPC windows against the oracle, the collective form through the library's own
NCCL communicator (q4_gpu_comm_*, unique id handed over by the host), and a peer that stops calling
between steps (host-side dropout, nothing in flight): the survivors' bounded wait reports it."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("world", [2, 4])
def test_fused_exchange_between_processes(world):
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    env = dict(os.environ, Q4_XCHG_TEST_DROPOUT="1", NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
           "--master-addr", "127.0.0.1", "--master-port", str(29600 + world), os.path.join(HERE, "xchg_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count(" ok") >= 8 * world + (world - 1)      # 6 fused + 2 collective calls per rank, dropout reports
