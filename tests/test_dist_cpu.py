"""Multi-process CPU tests over Gloo: the same algorithm / model code on a DistMesh, and
host-side failure detection (a rank that leaves, a rank that raises) without touching a GPU."""
import os
import re
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _launch(mode, nproc, port, timeout=240):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1", CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "dist_cpu_worker.py"), mode]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)


def test_algorithms_on_gloo_2x2_mesh():
    r = _launch("algorithms", 4, 29711)
    assert r.stdout.count("ALGORITHMS_OK") == 4, r.stdout + r.stderr[-2000:]


def test_model_step_on_gloo_matches_emulated_mesh():
    import torch
    from meshslice_b200.models.gpt import GPTConfig, GPTModel
    from meshslice_b200.parallel.mesh import EmuMesh, ShardedTensor
    r = _launch("model", 4, 29712)
    losses = [float(x) for x in re.findall(r"MODEL_LOSS ([0-9.]+)", r.stdout)]
    assert len(losses) == 4, r.stdout + r.stderr[-2000:]
    cfg = GPTConfig(n_layers=1, d_model=64, n_heads=4, ffn=256, vocab=300, seq=16, ksplits=(2, 2, 2, 2),
                    head_ksplit=2, vocab_pad=64, dtype=torch.float32)
    mesh = EmuMesh(2, 2)
    model = GPTModel(mesh, cfg)
    ids = torch.randint(0, cfg.vocab, (4, cfg.seq + 1), generator=torch.Generator().manual_seed(1))
    tok = ShardedTensor(mesh, {(r_, c): ids[r_ * 2:(r_ + 1) * 2, :-1].reshape(-1) for (r_, c) in mesh.coords()})
    tgt = ShardedTensor(mesh, {(r_, c): ids[r_ * 2:(r_ + 1) * 2, 1:].reshape(-1) for (r_, c) in mesh.coords()})
    loss = model.forward_backward(tok, tgt, 4 * cfg.seq)
    ref = (loss.shards[(0, 0)] + loss.shards[(1, 0)]).item()
    assert all(abs(l - ref) < 1e-4 for l in losses), (losses, ref)


def test_rank_leaving_between_steps_is_detected_before_the_next_collective():
    r = _launch("peer_leaves", 3, 29713)
    assert "rank 1 LEFT" in r.stdout
    assert r.stdout.count("PEER_LOST at step 3") == 2, r.stdout + r.stderr[-2000:]
    assert "UNEXPECTED_END" not in r.stdout


def test_rank_that_raises_tells_the_others():
    r = _launch("rank_raises", 2, 29714)
    assert "rank 0 RAISED" in r.stdout
    assert "rank 1 PEER_LOST" in r.stdout and "bad shard file" in r.stdout, r.stdout + r.stderr[-2000:]


def test_kernel_error_of_one_rank_raises_on_every_rank():
    r = _launch("status_agreement", 3, 29715)
    assert r.stdout.count("AGREED: kernel status 5 reported by rank 1") == 3, r.stdout + r.stderr[-2000:]
    assert "MISSED" not in r.stdout
