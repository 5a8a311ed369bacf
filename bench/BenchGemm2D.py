#!/usr/bin/env python
"""Single 2-D sharded GeMM sweep: fused MeshSlice OS / LS / RS kernels against the unsliced
NCCL + library-GEMM formulation, for several global shapes and slice counts on one mesh shape.

    torchrun --nproc-per-node 8 bench/BenchGemm2D.py --mesh 2x4 --slices 1 2 4 8 --json out.json

Per case it prints achieved TFLOP/s per GPU and the fraction of the roofline
max(FLOPs / measured GEMM peak, NVLink bytes / measured link bandwidth).  L2 is flushed before every
timed call; times are CUDA-event times on the launching stream, maximum over the ranks.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

SHAPES = [(16384, 4096, 16384), (16384, 16384, 4096), (16384, 12288, 49152), (16384, 49152, 12288)]  # M, K, N


_FLUSH = None


_ITERS, _WARM = 5, 3


def timeit(fn, iters=None, warm=None):
    """Mean device time of one call (CUDA events around every call on the launching stream, L2 flushed
    by a 256 MiB write before each, 3 warm-up calls), maximum over the ranks."""
    global _FLUSH
    iters, warm = iters or _ITERS, _WARM if warm is None else warm
    if _FLUSH is None:
        _FLUSH = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for e0, e1 in evs:
        _FLUSH.zero_()
        e0.record()
        fn()
        e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([sum(e0.elapsed_time(e1) for e0, e1 in evs) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item() * 1e-3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mesh", default="")
    ap.add_argument("--meshes", nargs="*", default=[], help="several RxC meshes in one job, e.g. 2x4 4x2 1x8 8x1")
    ap.add_argument("--slices", type=int, nargs="+", default=[1, 2, 4, 8])
    ap.add_argument("--shapes", type=int, nargs="*", default=[], help="M K N triples; default: the four headline shapes")
    ap.add_argument("--peak-tflops", type=float, default=1380.6)
    ap.add_argument("--link-gbs", type=float, default=770.0)
    ap.add_argument("--baselines", nargs="*", default=[], choices=["summa", "wang", "cannon"],
                    help="also time the OS product on these K-panel schedules")
    ap.add_argument("--sub", type=int, default=2, help="sub-panels per owner for --baselines")
    ap.add_argument("--iters", type=int, default=5, help="timed calls per case")
    ap.add_argument("--warm", type=int, default=3, help="warm-up calls per case (at least 3 for reported numbers)")
    ap.add_argument("--json", default="")
    args = ap.parse_args()
    global _ITERS, _WARM
    _ITERS, _WARM = args.iters, args.warm
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    from meshslice_b200.parallel import tensor_parallel as tp
    from meshslice_b200.parallel.engine import FusedEngine
    from meshslice_b200.parallel.mesh import DistMesh, ShardedTensor
    from meshslice_b200.trainer import choose_mesh

    mesh_specs = args.meshes or ([args.mesh] if args.mesh else ["%dx%d" % choose_mesh(world)])
    shapes = [tuple(args.shapes[i:i + 3]) for i in range(0, len(args.shapes), 3)] or SHAPES
    big = max(max(M * K, K * N, M * N) for M, K, N in shapes)
    out = []
    say = (lambda *a: print(*a, flush=True)) if rank == 0 else (lambda *a: None)
    for spec in mesh_specs:      # every mesh gets its own process groups, heap and engine, in one job
        R, C = [int(v) for v in spec.split("x")]
        mesh = DistMesh(R, C)
        eng = FusedEngine(mesh, 2 * big // R + (1 << 20), 2 * big // C + (1 << 20), 2 * big // min(R, C) + (1 << 20))
        run_mesh(args, mesh, eng, shapes, world, out, say, tp, ShardedTensor)
        torch.cuda.empty_cache()
    if rank == 0 and args.json:
        json.dump(out, open(args.json, "w"), indent=1)
    dist.barrier()
    dist.destroy_process_group()


def run_mesh(args, mesh, eng, shapes, world, out, say, tp, ShardedTensor):
    R, C = mesh.R, mesh.C
    key = (mesh.r, mesh.c)
    for (M, K, N) in shapes:
        flops = 2.0 * M * K * N / world
        t_comp = flops / (args.peak_tflops * 1e12)
        # operands per dataflow (local shards), drawn on the device; weights placed in the heap
        def rnd(a, b):
            return torch.randn(a, b, device="cuda").bfloat16()
        cases = {
            "os": (rnd(M // R, K // C), rnd(K // R, N // C), ((C - 1) * (M // R) * (K // C) + (R - 1) * (K // R) * (N // C)) * 2),
            "ls": (rnd(M // R, K // C), rnd(N // R, K // C), ((R - 1) * (N // R) * (K // C) + (C - 1) * (M // R) * (N // C)) * 2),
            "rs": (rnd(K // R, M // C), rnd(K // R, N // C), ((C - 1) * (K // R) * (M // C) + (R - 1) * (M // R) * (N // C)) * 2),
        }
        for df, (x, w, link_bytes) in cases.items():
            roof = max(t_comp, link_bytes / (args.link_gbs * 1e9))
            xs, ws = ShardedTensor(mesh, {key: x}), ShardedTensor(mesh, {key: w})
            base_fn = {"os": tp.collective_os, "ls": tp.collective_ls, "rs": tp.collective_rs}[df]
            t_base = timeit(lambda: base_fn(mesh, xs, ws))
            row = dict(M=M, K=K, N=N, mesh=[R, C], dataflow=df, nccl_cublas_ms=t_base * 1e3,
                       nccl_cublas_tflops=flops / t_base / 1e12, roofline_ms=roof * 1e3, fused={})
            for s in args.slices:
                fn = getattr(eng, df)
                t = timeit(lambda: fn(x, w, n_slices=s))
                eng.check()
                row["fused"][s] = dict(ms=t * 1e3, tflops=flops / t / 1e12, roofline_frac=roof / t,
                                       speedup_vs_nccl=t_base / t)
            if df == "os" and args.baselines:
                # SUMMA / Wang / Cannon on the same kernel: K panels consumed in that algorithm's order
                row["k_panel"] = {}
                for order in args.baselines:
                    if order == "cannon" and R != C:
                        continue
                    t = timeit(lambda: eng.os_kpanel(x, w, order=order, sub=args.sub))
                    eng.check()
                    row["k_panel"][order] = dict(ms=t * 1e3, tflops=flops / t / 1e12, roofline_frac=roof / t)
            say(json.dumps(row))
            out.append(row)


if __name__ == "__main__":
    main()
