"""Fused compute+collective kernels on 2 GPUs of one node (skipped with fewer)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.timeout(600)
def test_fused_collectives_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", GFS_SYMM_CANARIES="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29561", os.path.join(here, "fused_comm_worker.py")]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=540)
    tail = (proc.stdout + "\n" + proc.stderr)[-4000:]
    assert proc.returncode == 0 and "WORKER OK" in proc.stdout, tail
