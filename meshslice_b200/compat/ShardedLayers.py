"""Names of ShardedLayers.py mapped to this package."""
from ..models.sharded_layers import (ShardedAttention, ShardedFFLayer, ShardedLayerNorm,  # noqa: F401
                                     TransformerBlock)


def main(argv=None):
    """The block benchmark of ShardedLayers.py:192-235: build one TransformerBlock with dataflows
    os / os / os / ls, run forward and backward, print the time per pass.

    Under ``torchrun`` on GPUs the mesh is the job's 2-D mesh with the fused engine attached
    (``--nrows`` x ``--ncols``, GPT-3 sizes by default); started as a single process it runs a
    small block on an emulated 2 x 2 mesh on the CPU, which checks the plumbing, not the speed."""
    import argparse
    import os
    import time

    import torch

    from ..parallel.mesh import EmuMesh
    from ..parallel.tensor_parallel import createMultihostMatrix
    p = argparse.ArgumentParser()
    p.add_argument("alg", nargs="?", default="meshflow")
    p.add_argument("--nrows", type=int, default=2)
    p.add_argument("--ncols", type=int, default=2)
    p.add_argument("--iters", type=int, default=10)
    a = p.parse_args(argv)
    distributed = "RANK" in os.environ and torch.cuda.is_available()
    if distributed:
        import torch.distributed as dist

        from ..parallel.engine import FusedEngine
        from ..parallel.mesh import DistMesh
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
        dist.init_process_group("nccl")
        B, S, H, D = 32, 2048, 96, 128
        mesh = DistMesh(a.nrows, a.ncols)
        dev = torch.device("cuda")
        T, d = B * S, H * D
        m = T // mesh.R
        FusedEngine(mesh, m * 4 * d * 2 + (1 << 20), 4 * d * d // mesh.C * 2 + (1 << 20),
                    max(m * 4 * d, 4 * d * d // min(mesh.R, mesh.C)) * 2 + (1 << 20), exchange_rows=m)
        rank0 = dist.get_rank() == 0
    else:
        B, S, H, D = 4, 128, 8, 64
        mesh, dev, rank0 = EmuMesh(a.nrows, a.ncols), torch.device("cpu"), True
    block = TransformerBlock(mesh, S, H, D, ["os", "os", "os", "ls"], alg=a.alg, device=dev, std=0.02)
    x = createMultihostMatrix(mesh, (B * S, H * D), device=dev, seed=11)
    dy = createMultihostMatrix(mesh, (B * S, H * D), device=dev, seed=12)

    def sync():
        if dev.type == "cuda":
            torch.cuda.synchronize()

    block.forward(x)
    block.backward(dy)
    sync()
    t0 = time.time()
    for _ in range(a.iters):
        block.forward(x)
    sync()
    t1 = time.time()
    for _ in range(a.iters):
        block.forward(x)
        block.backward(dy)
    sync()
    t2 = time.time()
    if rank0:
        fwd = (t1 - t0) / a.iters * 1e3
        print(f"forward {fwd:.3f} ms, forward+backward {(t2 - t1) / a.iters * 1e3:.3f} ms "
              f"({a.alg}, mesh {mesh.R}x{mesh.C}, B={B} S={S} H={H} D={D})")
    if distributed:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
