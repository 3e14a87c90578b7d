"""GPU, two or more devices: the batch-sharded forward over NCCL returns, on every rank, ids bit-identical to the
single-GPU forward of the whole batch.  Skipped on a one-GPU box (the gloo tests cover the host logic there)."""

import os
import subprocess
import sys

import pytest
import torch

from conftest import ROOT

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
def test_sharded_forward_over_nccl_matches_single_gpu():
    n = min(torch.cuda.device_count(), 4)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(n), "--master-addr", "127.0.0.1",
                          "--master-port", "29611", os.path.join(ROOT, "tests", "sharded_nccl_worker.py")],
                         capture_output=True, text=True, timeout=900, cwd=ROOT, env=env)
    assert res.returncode == 0, (res.stdout[-2000:], res.stderr[-4000:])
    assert f"sharded_nccl_worker ok: world {n}" in res.stdout
