#!/usr/bin/env python
"""Exhaustive (mesh shape x slice count) grid of the transformer block's four sharded linears
(forward + backward, fused MeshSlice kernels) inside ONE job, next to the autotuner's prediction
and pick for the same block.  Answers "is the tuner's choice within x % of the best measured
configuration" on this box.

    torchrun --nproc-per-node 8 bench/BenchMeshGrid.py --fabric-json fabric.json --json grid.json
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--batchsize", type=int, default=32)
    p.add_argument("--seqlen", type=int, default=2048)
    p.add_argument("--nheads", type=int, default=32)
    p.add_argument("--headdim", type=int, default=128)
    p.add_argument("--meshes", nargs="*", default=[])
    p.add_argument("--slices", type=int, nargs="+", default=[1, 4])
    p.add_argument("--iters", type=int, default=3)
    p.add_argument("--fabric-json", default="")
    p.add_argument("--json", default="")
    a = p.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    from meshslice_b200 import autotuner as AT
    from meshslice_b200.models.sharded_layers import ShardedFFLayer
    from meshslice_b200.parallel.engine import FusedEngine
    from meshslice_b200.parallel.mesh import DistMesh
    from meshslice_b200.parallel.tensor_parallel import createMultihostMatrix

    B, S, H, D = a.batchsize, a.seqlen, a.nheads, a.headdim
    T, d = B * S, H * D
    meshes = [tuple(int(v) for v in m.split("x")) for m in a.meshes] or AT.candidate_shapes(world)
    dev = torch.device("cuda")
    rows = []
    for (R, C) in meshes:
        if T % (R * 256) or d % (C * 256) or (T // R) % 256:
            continue
        mesh = DistMesh(R, C)
        m = T // R
        eng = FusedEngine(mesh, m * 4 * d * 2 + (1 << 20), 4 * d * d // C * 2 + (1 << 20),
                          max(m * 4 * d, 4 * d * d // min(R, C)) * 2 + (1 << 20), exchange_rows=m)
        for k in a.slices:
            kw = dict(device=dev, std=0.02)
            layers = [ShardedFFLayer(mesh, "meshslice", "ls", k, d, d, seed=1, **kw),
                      ShardedFFLayer(mesh, "meshslice", "os", k, d, 4 * d, seed=2, **kw),
                      ShardedFFLayer(mesh, "meshslice", "ls", k, 4 * d, d, seed=3, **kw),
                      ShardedFFLayer(mesh, "meshslice", "os", k, d, 3 * d, seed=4, **kw)]
            x = createMultihostMatrix(mesh, (T, d), device=dev, seed=5)
            dy = createMultihostMatrix(mesh, (T, 3 * d), device=dev, seed=6)
            def step():
                h = x
                for l in layers:
                    h = l.forward(h)
                g = dy
                for l in reversed(layers):
                    g = l.backward(g)
            step()
            eng.check()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(a.iters):
                step()
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / a.iters], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            eng.check()
            flops = 3 * 2.0 * T * 12 * d * d
            rows.append(dict(mesh=[R, C], ksplit=k, ms=t.item(), tflops_per_gpu=flops / world / (t.item() * 1e-3) / 1e12))
            if rank == 0:
                print(json.dumps(rows[-1]), flush=True)
            del layers, x, dy
            torch.cuda.empty_cache()
    if rank == 0:
        fabric = (AT.FabricConstants.load(a.fabric_json) if a.fabric_json else AT.FabricConstants.from_dict(AT.B200_NVSWITCH))
        graph = AT.build_transformerBlock(B, S, H, D)
        tuner = AT.Autotuner(graph, [tuple(r["mesh"]) for r in rows if r["ksplit"] == a.slices[0]], fabric=fabric,
                             blocksize=64, klist=a.slices, verbose=False)
        tuner.emulatedFinetune(sweep=True)
        best = min(rows, key=lambda r: r["ms"])
        pick = list(tuner.bestshape)
        pick_rows = [r for r in rows if r["mesh"] == pick]
        pick_ms = min(r["ms"] for r in pick_rows) if pick_rows else None
        out = dict(grid=rows, best_measured=best, tuner_pick=tuner.result(),
                   tuner_pick_measured_ms=pick_ms, pick_over_best=(pick_ms / best["ms"]) if pick_ms else None)
        print(json.dumps({k: v for k, v in out.items() if k != "grid"}), flush=True)
        if a.json:
            json.dump(out, open(a.json, "w"), indent=1)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
