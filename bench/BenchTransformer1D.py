#!/usr/bin/env python
"""1-D baselines with the reference's flags (BenchTransformer1D.py:122-128): tensor parallel
(Wang collective-matmul OS / IS) or FSDP over a 1 x n mesh, linear layers or (``--noff``) the
non-linear ops.  Runs on the GPUs launched by torchrun (NCCL collectives + library GEMM), or on
an emulated CPU mesh of ``--ndev`` devices when started without torchrun.
"""
import argparse
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--batchsize", type=int, default=-1)
    p.add_argument("--seqlen", type=int, default=2048)
    p.add_argument("--nheads", type=int, default=96)
    p.add_argument("--headdim", type=int, default=128)
    p.add_argument("--alg", type=str, default="tp", choices=["tp", "fsdp"])
    p.add_argument("--noff", action="store_true")
    p.add_argument("--ndev", type=int, default=4)
    p.add_argument("--iters", type=int, default=3)
    a = p.parse_args()
    world = int(os.environ.get("WORLD_SIZE", 1))
    from meshslice_b200.models.sharded_layers import GeLU, ShardedAttention, ShardedLayerNorm
    from meshslice_b200.parallel.mesh import DistMesh, EmuMesh, ShardedTensor
    from meshslice_b200.parallel.tensor_parallel_1d import SPMDWang, createShardedMatrix
    if world > 1:
        import torch.distributed as dist
        rank = int(os.environ["RANK"])
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
        mesh, n, dev = DistMesh(1, world), world, torch.device("cuda")
        dtype = torch.bfloat16
    else:
        rank, n, dev, dtype = 0, a.ndev, None, torch.float32
        mesh = EmuMesh(1, n)
        a.seqlen, a.nheads = min(a.seqlen, 128), min(a.nheads, 8)   # keep the CPU emulation small
    B = n if a.batchsize <= 0 else a.batchsize
    S, H, D = a.seqlen, a.nheads, a.headdim
    T, d = B * S, H * D
    sp = SPMDWang(mesh)
    def rows(full_shape, seed):
        st = createShardedMatrix(mesh, full_shape, dtype=dtype, shard_axis=0, seed=seed, device=dev)
        return st
    def cols(full_shape, seed):
        return createShardedMatrix(mesh, full_shape, dtype=dtype, shard_axis=1, seed=seed, device=dev)
    if a.noff:
        if a.alg == "tp":       # heads split over devices, LayerNorm statistics all-reduced
            m2 = mesh
            x = cols((T, 3 * d), 1)
            attn, norm, gelu = ShardedAttention(m2, H, S), ShardedLayerNorm(m2, d, dtype=dtype, device=dev), GeLU()
            fn = lambda: norm.forward(gelu.forward(norm.forward(attn.forward(x))))
        else:                   # batch split: everything local
            m2 = EmuMesh(n, 1) if world == 1 else DistMesh(world, 1)
            x = ShardedTensor(m2, {k: v for k, v in zip(m2.coords(), rows((T, 3 * d), 1).shards.values())})
            attn, norm, gelu = ShardedAttention(m2, H, S), ShardedLayerNorm(m2, d, dtype=dtype, device=dev), GeLU()
            fn = lambda: norm.forward(gelu.forward(norm.forward(attn.forward(x))))
        flops = 0.0
    elif a.alg == "tp":
        x, w1, w2 = cols((T, d), 1), cols((d, 4 * d), 2), cols((d, 4 * d), 3)
        fn = lambda: sp.IS(sp.OS(x, w1), w2)          # ff1 (column-parallel) then ff2 (row-parallel)
        flops = 2.0 * T * 8 * d * d
    else:
        x, w1, w2 = rows((T, d), 1), cols((d, 4 * d), 2), cols((4 * d, d), 3)
        fn = lambda: sp.DP(sp.DP(x, w1), w2)
        flops = 2.0 * T * 8 * d * d
    fn()
    if dev is not None:
        torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(a.iters):
        fn()
    if dev is not None:
        torch.cuda.synchronize()
    ms = (time.perf_counter() - t0) / a.iters * 1e3
    if rank == 0:
        out = {"alg": a.alg, "noff": a.noff, "ndev": n, "forward_ms": ms}
        if flops and dev is not None:
            out["tflops_per_gpu"] = flops / n / (ms * 1e-3) / 1e12
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
