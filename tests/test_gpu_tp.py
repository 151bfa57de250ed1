"""Tensor-parallel row shards with the fused all-reduce, on 2+ GPUs of one node."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_allreduce_row_parallel_parity():
    c = torch.cuda.device_count()
    world = 8 if c >= 8 else 4 if c >= 4 else 2        # every GPU of the box, as 2, 4 or 8 ranks
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", "29541", os.path.join(ROOT, "tests", "tp_worker.py")]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert "TP_PARITY_OK" in out.stdout, out.stdout[-3000:] + out.stderr[-3000:]
