#!/usr/bin/env python
"""Transformer-block benchmark with the reference's flags (BenchTransformer.py:23-30):
four chained sharded linears (out_proj 'ls' -> ff1 'os' -> ff2 'ls' -> in_proj 'os') forward and
backward, or with ``--alg noff`` the non-linear ops only (attention, three LayerNorms, two adds,
GeLU).  Unlike the reference, which only writes a profiler trace, this prints device-timed
forward / backward milliseconds (max over ranks) and achieved TFLOP/s per GPU.

    torchrun --nproc-per-node 8 bench/BenchTransformer.py --alg meshflow --nrows 2 --ncols 4

``--nrows x --ncols`` is the LOGICAL mesh of the study.  When fewer GPUs are launched than it has
devices, the physical mesh (``--phys RxC``, default: the most square split of the launched ranks
that divides the logical one) runs the per-device problem of the logical mesh, the reference's
weak-scaling emulation (BenchTransformer.py:45-56,78-79): batch * phys_rows / nrows sequences and
heads * phys_cols / ncols heads, so every GPU holds the shards and does the FLOPs it would in the
large run; only the collective group sizes are those of the physical mesh.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def physical_mesh(nrows: int, ncols: int, world: int, phys: str = ""):
    """Physical mesh for a logical nrows x ncols study on ``world`` ranks: the logical mesh itself
    when the ranks suffice, else ``phys`` or the most square split whose sides divide the logical ones."""
    if phys:
        pr, pc = (int(v) for v in phys.lower().split("x"))
    elif nrows * ncols == world:
        return nrows, ncols
    else:
        cands = [(r, world // r) for r in range(1, world + 1)
                 if world % r == 0 and nrows % r == 0 and ncols % (world // r) == 0]
        if not cands:
            raise SystemExit(f"no split of {world} ranks divides the logical mesh {nrows}x{ncols}")
        pr, pc = min(cands, key=lambda rc: abs(rc[0] - rc[1]))
    if pr * pc != world or nrows % pr or ncols % pc:
        raise SystemExit(f"physical mesh {pr}x{pc} does not match {world} ranks / logical mesh {nrows}x{ncols}")
    return pr, pc


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--ksplit", nargs=4, type=int, default=[8, 8, 8, 8], help="slice count per linear layer")
    p.add_argument("--batchsize", type=int, default=-1, help="default: number of chips")
    p.add_argument("--seqlen", type=int, default=2048)
    p.add_argument("--nheads", type=int, default=96, help="gpt3: 96, megatron: 160")
    p.add_argument("--headdim", type=int, default=128)
    p.add_argument("--nrows", type=int, default=2)
    p.add_argument("--ncols", type=int, default=4)
    p.add_argument("--alg", type=str, default="noff", choices=["noff", "collective", "cannon", "wang", "meshflow", "summa"])
    p.add_argument("--iters", type=int, default=3)
    p.add_argument("--phys", default="", help="physical mesh RxC when it is smaller than --nrows x --ncols")
    a = p.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    from meshslice_b200.models.sharded_layers import (GeLU, ShardedAttention, ShardedFFLayer, ShardedLayerNorm, _add)
    from meshslice_b200.parallel.engine import FusedEngine, LocalGemmEngine
    from meshslice_b200.parallel.mesh import DistMesh, EmuMesh
    from meshslice_b200.parallel.tensor_parallel import createMultihostMatrix

    pr, pc = physical_mesh(a.nrows, a.ncols, world, a.phys)
    B_log = a.nrows * a.ncols if a.batchsize <= 0 else a.batchsize
    if (B_log * pr) % a.nrows or (a.nheads * pc) % a.ncols:
        raise SystemExit("batch / heads of the logical mesh do not scale to the physical one")
    # per-device problem of the logical mesh on the physical one
    B, H = B_log * pr // a.nrows, a.nheads * pc // a.ncols
    S, D = a.seqlen, a.headdim
    mesh = DistMesh(pr, pc) if world > 1 else EmuMesh(1, 1)
    dev = torch.device("cuda")
    T, d = B * S, H * D
    if a.alg != "noff" and a.alg != "collective":
        if world > 1:
            m = T // pr
            FusedEngine(mesh, m * 4 * d * 2, 4 * d * d // pc * 2 + (1 << 20), m * 4 * d * 2 + (1 << 20),
                        exchange_rows=m)
        else:
            LocalGemmEngine(mesh)

    def sync_time(fn):
        fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / a.iters], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    tag = "{}_{}x{}_{}_{}_{}".format(a.alg, a.nrows, a.ncols, B_log, a.nheads, D)
    if a.alg == "noff":
        x0 = createMultihostMatrix(mesh, (T, 3 * d), device=dev)
        norm, attn, gelu = ShardedLayerNorm(mesh, d, device=dev), ShardedAttention(mesh, H, S), GeLU()
        norm2, norm3 = ShardedLayerNorm(mesh, d, device=dev), ShardedLayerNorm(mesh, d, device=dev)
        def fwd():
            res = attn.forward(x0)
            out = norm.forward(res)
            res2 = norm2.forward(res, out)
            out = gelu.forward(res2)
            return norm3.forward(res2, out)
        dy = createMultihostMatrix(mesh, (T, d), device=dev, seed=9)
        def bwd():
            fwd()
            g3 = norm3.backward(dy)
            g2 = norm2.backward(_add(gelu.backward(g3), g3))
            return attn.backward(_add(norm.backward(g2), g2))
        tf, tb = sync_time(fwd), sync_time(bwd)
        flops = 0.0
    else:
        alg = "meshslice" if a.alg == "meshflow" else a.alg
        kw = dict(device=dev, std=0.02)
        out_proj = ShardedFFLayer(mesh, alg, "ls", a.ksplit[1], d, d, seed=1, **kw)
        ff1 = ShardedFFLayer(mesh, alg, "os", a.ksplit[2], d, 4 * d, seed=2, **kw)
        ff2 = ShardedFFLayer(mesh, alg, "ls", a.ksplit[3], 4 * d, d, seed=3, **kw)
        in_proj = ShardedFFLayer(mesh, alg, "os", a.ksplit[0], d, 3 * d, seed=4, **kw)
        x = createMultihostMatrix(mesh, (T, d), device=dev, seed=5)
        dy = createMultihostMatrix(mesh, (T, 3 * d), device=dev, seed=6)
        layers = [out_proj, ff1, ff2, in_proj]
        def fwd():
            h = x
            for l in layers:
                h = l.forward(h)
            return h
        def bwd():
            fwd()
            g = dy
            for l in reversed(layers):
                g = l.backward(g)
            return g
        tf, tb = sync_time(fwd), sync_time(bwd)
        flops = 2.0 * T * (d * d + 4 * d * d + 4 * d * d + 3 * d * d)
    if rank == 0:
        tb_only = tb - tf
        out = {"benchtag": tag, "logical_mesh": [a.nrows, a.ncols], "physical_mesh": [pr, pc],
               "batch_run": B, "heads_run": H, "forward_ms": tf, "backward_ms": tb_only, "fwd_bwd_ms": tb}
        if flops:
            out["tflops_per_gpu_fwd"] = flops / world / (tf * 1e-3) / 1e12
            out["tflops_per_gpu_fwd_bwd"] = 3 * flops / world / (tb * 1e-3) / 1e12
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
