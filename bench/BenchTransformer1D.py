#!/usr/bin/env python
"""1-D baselines with the reference's flags (BenchTransformer1D.py:122-128): tensor parallel (Wang
collective matmul, 'os' / 'is' layers) or FSDP, either the four chained linear layers of a block
(out_proj, ff1, ff2, in_proj) or, with ``--noff``, the non-linear ops (attention, three LayerNorms,
two adds, GeLU).  Forward AND backward are timed, on the device, maximum over the ranks.

    torchrun --nproc-per-node 8 bench/BenchTransformer1D.py --alg tp            # 1 x 8, fused kernels
    torchrun --nproc-per-node 8 bench/BenchTransformer1D.py --alg fsdp --noff
    python bench/BenchTransformer1D.py --ndev 4                                 # emulated CPU mesh, small

``--ndev`` scales the per-device sizes to those of a larger machine as the reference does
(BenchTransformer1D.py:131,146,168): with n devices present, tensor parallelism keeps heads *
n / ndev per device, FSDP keeps batch * n / ndev.
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
    p.add_argument("--batchsize", type=int, default=-1, help="default: number of devices")
    p.add_argument("--seqlen", type=int, default=2048)
    p.add_argument("--nheads", type=int, default=96)
    p.add_argument("--headdim", type=int, default=128)
    p.add_argument("--alg", type=str, default="tp", choices=["tp", "fsdp"])
    p.add_argument("--noff", action="store_true")
    p.add_argument("--ndev", type=int, default=0, help="device count to extrapolate to (default: the devices present)")
    p.add_argument("--iters", type=int, default=3)
    p.add_argument("--backend", default="fused", choices=["fused", "collective"])
    a = p.parse_args()
    world = int(os.environ.get("WORLD_SIZE", 1))
    from meshslice_b200.models.sharded_layers import GeLU, _add
    from meshslice_b200.models.sharded_layers_1d import ShardedAttention1D, ShardedFFLayer1D, ShardedLayerNorm1D
    from meshslice_b200.parallel.mesh import DistMesh, EmuMesh
    from meshslice_b200.parallel.tensor_parallel import createMultihostMatrix
    gpu = world > 1 or (torch.cuda.is_available() and a.ndev == 0)
    if world > 1:
        import torch.distributed as dist
        rank = int(os.environ["RANK"])
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
        n, dev, dtype = world, torch.device("cuda"), torch.bfloat16
    elif gpu:
        rank, n, dev, dtype = 0, 1, torch.device("cuda"), torch.bfloat16
    else:
        rank, n, dev, dtype = 0, a.ndev or 4, None, torch.float32
        a.seqlen, a.nheads, a.headdim = min(a.seqlen, 64), min(a.nheads, 8), min(a.headdim, 16)
    ndev = a.ndev or n
    B = ndev if a.batchsize <= 0 else a.batchsize
    S, H, D = a.seqlen, a.nheads, a.headdim
    tp = a.alg == "tp"
    R, C = (1, n) if tp else (n, 1)
    B2, H2 = (B, H * n // ndev) if tp else (B * n // ndev, H)      # per-device sizes of the ndev-device run
    if world > 1:
        mesh = DistMesh(R, C)
    else:
        mesh = EmuMesh(R, C)
    T, d, d2 = B2 * S, H * D, H2 * D
    if gpu:
        from meshslice_b200.parallel.engine import FusedEngine, LocalGemmEngine
        if world > 1 and a.backend == "fused":
            m = T // R
            FusedEngine(mesh, m * 4 * d2 * 2 + (1 << 20), 4 * d * d2 // C * 2 + (1 << 20),
                        max(m * 4 * d2, 4 * d * d2 // min(R, C)) * 2 + (1 << 20), exchange_rows=m)
        elif world == 1:
            LocalGemmEngine(mesh)
    kw = dict(dtype=dtype, device=dev, std=0.02)
    if a.noff:
        sharding = "tp" if tp else "dp"
        x = createMultihostMatrix(mesh, (T, 3 * d2), device=dev, seed=1, dtype=dtype)
        dy = createMultihostMatrix(mesh, (T, d2), device=dev, seed=2, dtype=dtype)
        attn = ShardedAttention1D(mesh, H2, S, sharding, allow_fallback=not gpu or D != 128)
        n1, n2, n3 = (ShardedLayerNorm1D(mesh, d2, sharding, dtype=dtype, device=dev) for _ in range(3))
        gelu = GeLU()

        def forward():          # attention, three norms, two adds, one GeLU (BenchTransformer1D.py:150-156)
            res = attn.forward(x)
            out = n1.forward(res)
            res2 = n2.forward(res, out)              # LN(res + out)
            out = gelu.forward(res2)
            return n3.forward(res2, out)             # LN(res2 + out)

        def backward():
            d3 = n3.backward(dy)                     # gradient of res2 + gelu(res2)
            d2_ = n2.backward(_add(gelu.backward(d3), d3))
            return attn.backward(_add(n1.backward(d2_), d2_))
        flops = 0.0
    else:
        df = ("is", "os", "is", "os") if tp else ("fsdp",) * 4
        dims = [(d2, d), (d, 4 * d2), (4 * d2, d), (d, 3 * d2)]      # out_proj, ff1, ff2, in_proj
        if not tp:
            dims = [(d, d), (d, 4 * d), (4 * d, d), (d, 3 * d)]
        layers = [ShardedFFLayer1D(mesh, f, i, o, seed=11 + j, backend="auto" if a.backend == "fused" else "collective",
                                   **kw) for j, (f, (i, o)) in enumerate(zip(df, dims))]
        x = createMultihostMatrix(mesh, (T, dims[0][0]), device=dev, seed=1, dtype=dtype)
        dy = createMultihostMatrix(mesh, (T, dims[-1][1]), device=dev, seed=2, dtype=dtype)

        def forward():
            out = x
            for l in layers:
                out = l.forward(out)
            return out

        def backward():
            g = dy
            for l in reversed(layers):
                g = l.backward(g)
            return g
        flops = sum(2.0 * T * i * o for i, o in dims)        # forward FLOPs of the whole mesh

    def timed(fn):
        if dev is None:
            t0 = time.perf_counter()
            for _ in range(a.iters):
                fn()
            return (time.perf_counter() - t0) / a.iters * 1e3
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0.record()
        for _ in range(a.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1) / a.iters], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item()

    forward()
    backward()
    fwd_ms = timed(forward)
    forward()
    bwd_ms = timed(lambda: (forward(), backward()))     # backward needs a fresh forward: difference below
    bwd_ms = max(bwd_ms - fwd_ms, 0.0)
    if gpu:
        from meshslice_b200 import _native
        _native.check_status()
    if rank == 0:
        out = {"alg": a.alg, "noff": a.noff, "devices": n, "ndev": ndev, "batch": B2, "heads": H2,
               "forward_ms": fwd_ms, "backward_ms": bwd_ms,
               "timing": "device events, max over ranks" if dev is not None else "host clock (CPU emulation)"}
        if flops and dev is not None:
            # forward + backward (dX and dW) = 3x the forward FLOPs, split evenly over the devices
            out["tflops_per_gpu"] = 3.0 * flops / n / ((fwd_ms + bwd_ms) * 1e-3) / 1e12
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
