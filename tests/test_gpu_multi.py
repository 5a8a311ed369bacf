"""Fused kernels across real GPUs: runs only where at least two are visible.  One process per GPU
under torchrun; every wait in the kernels is bounded, so a failure ends as an error status."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

_HERE = os.path.dirname(os.path.abspath(__file__))


def _run_worker(nproc, mesh, slices, port):
    env = dict(os.environ, MESH=mesh, SLICES=str(slices), MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(_HERE, "dist_fused_worker.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=420)
    assert res.returncode == 0 and "FUSED_MULTI_GPU_OK" in res.stdout, (res.stdout[-2000:], res.stderr[-2000:])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_dataflows_on_two_gpus():
    _run_worker(2, "1x2", 2, 29731)
    _run_worker(2, "2x1", 2, 29732)


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs four GPUs")
def test_fused_dataflows_on_a_2x2_mesh():
    _run_worker(4, "2x2", 2, 29733)
