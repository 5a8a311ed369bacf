#!/usr/bin/env python
"""Row / column all-gather, reduce-scatter and send-recv sweep on the GPUs of one box, for the
NCCL collectives and for the in-kernel peer-to-peer collectives of this package; fits the cost
model's fabric constants and writes them as JSON.

Counterpart of BenchCollectives2D.py (same positional argument: allgather | reducescatter |
sendrecv | all; sizes are per-device shard sizes, bf16).  Launch with torchrun, one rank per GPU:

    torchrun --nproc-per-node 8 bench/BenchCollectives2D.py all --mesh 2x4 --fabric-json fabric.json

Timing: CUDA events on the launching stream after warm-up, max over ranks.
"""
import argparse
import json
import os
import sys
from statistics import mean, stdev

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def repeat_bench(fn, repeat=5, inner=10, warmup=5):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    times = []
    for _ in range(repeat):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(inner):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / inner], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        times.append(t.item() * 1e-3)
    return times


def fit_line(sizes, times):
    """Least squares t = a + b * bytes on the upper half of the sweep (bandwidth regime) and the
    intercept from the smallest sizes (latency regime)."""
    import numpy as np
    s, t = np.array(sizes, dtype=float), np.array(times, dtype=float)
    hi = s >= np.median(s)
    b = np.polyfit(s[hi], t[hi], 1)[0]
    a = float(t[:3].mean())
    return a, float(b)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("which", nargs="?", default="all", choices=["allgather", "reducescatter", "sendrecv", "all"])
    ap.add_argument("--mesh", default="")
    ap.add_argument("--min-bytes", type=int, default=1 << 10)
    ap.add_argument("--max-bytes", type=int, default=1 << 30, help="largest per-device shard (default 1 GiB)")
    ap.add_argument("--fabric-json", default="")
    ap.add_argument("--impl", default="both", choices=["nccl", "p2p", "both"])
    ap.add_argument("--p2p-mode", default="push", choices=["push", "pull"],
                    help="all-gather / send-recv of the P2P twins: posted stores to the peers, or loads from them")
    args = ap.parse_args()

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    from meshslice_b200 import _native
    from meshslice_b200.parallel import runtime as rt
    from meshslice_b200.parallel.collectives import P2PCollectives
    from meshslice_b200.parallel.mesh import DistMesh, ShardedTensor
    from meshslice_b200.trainer import choose_mesh

    R, C = [int(v) for v in args.mesh.split("x")] if args.mesh else choose_mesh(world)
    mesh = DistMesh(R, C)
    heap = rt.SymmHeap(args.max_bytes * (1 + (max(R, C) if args.p2p_mode == "push" else 0)) + (16 << 20))
    p2p = P2PCollectives(mesh, heap, args.max_bytes)
    sizes = []
    b = args.min_bytes
    while b <= args.max_bytes:
        sizes.append(b)
        b *= 4
    kinds = ["allgather", "reducescatter", "sendrecv"] if args.which == "all" else [args.which]
    results = []
    say = (lambda *a: print(*a, flush=True)) if rank == 0 else (lambda *a: None)
    say(f"Running benchmark on {(R, C)} devices.")
    for kind in kinds:
        for axis, n in (("col", C), ("row", R)):
            if n == 1:
                continue
            for dim in ((0, 1) if kind != "sendrecv" else (0,)):
                for impl in (["nccl", "p2p"] if args.impl == "both" else [args.impl]):
                    say(f"\n{kind}_{axis} dim={dim} [{impl}]")
                    for nbytes in sizes:
                        cols = 512 if nbytes >= 1024 * 8 else 64
                        rows = max(n if kind == "reducescatter" else 1, nbytes // (cols * 2))
                        if kind == "reducescatter":
                            rows = (rows + n - 1) // n * n
                            cols = (cols + 8 * n - 1) // (8 * n) * (8 * n)
                        x = p2p.input((rows, cols))
                        x.normal_()
                        st = ShardedTensor(mesh, {(mesh.r, mesh.c): x})
                        if impl == "nccl":
                            fn = {"allgather": lambda: mesh.all_gather(st, axis, dim),
                                  "reducescatter": lambda: mesh.reduce_scatter(st, axis, dim),
                                  "sendrecv": lambda: mesh.permute(st, axis, 1)}[kind]
                        else:
                            push = args.p2p_mode == "push"
                            fn = {"allgather": lambda: p2p.all_gather(rows, cols, axis, dim, push=push),
                                  "reducescatter": lambda: p2p.reduce_scatter(rows, cols, axis, dim),
                                  "sendrecv": lambda: p2p.send_recv(rows, cols, axis, push=push)}[kind]
                        ts = repeat_bench(fn, repeat=3 if nbytes >= (1 << 26) else 5, inner=3 if nbytes >= (1 << 26) else 10)
                        _native.check_status()
                        actual = rows * cols * 2
                        say("Size: {}KB,\t Time: {:.4f}+-{:.4f}ms".format(actual // 1024, mean(ts) * 1e3,
                                                                           (stdev(ts) if len(ts) > 1 else 0) * 1e3))
                        results.append(dict(kind=kind, axis=axis, dim=dim, impl=impl, bytes=actual, n=n, t=mean(ts)))
    if rank == 0 and args.fabric_json:
        lat, bws, base = {}, {}, {}
        use = "p2p" if args.impl != "nccl" else "nccl"
        for kind in ("allgather", "reducescatter", "sendrecv"):
            per_axis = {}
            for axis, n in (("row", R), ("col", C)):
                rs = [r for r in results if r["kind"] == kind and r["axis"] == axis and r["impl"] == use and r["dim"] == 0]
                if not rs:
                    continue
                a, b = fit_line([r["bytes"] for r in rs], [r["t"] for r in rs])
                moved = (n - 1) if kind != "sendrecv" else 1
                if kind == "reducescatter":
                    moved = (n - 1) / n
                per_axis[axis] = (a, moved / b if b > 0 else float("inf"))
            if not per_axis:
                continue
            a0 = min(v[0] for v in per_axis.values())
            lat[kind] = min(a0 / 2, 5e-6)
            base[kind] = max(a0 - lat[kind], 0.0)
            row_bw = per_axis.get("row", per_axis.get("col"))[1]
            col_bw = per_axis.get("col", per_axis.get("row"))[1]
            bws[kind] = [row_bw, col_bw]      # (mesh dim 0 = rows, mesh dim 1 = columns)
        peaks = {}
        json.dump(dict(latencies=lat, bws=bws, base_overheads=base, fabric="switch", shared_port=True,
                       flops_per_chip=1.38e15, mesh=[R, C], impl=use, samples=results), open(args.fabric_json, "w"), indent=1)
        say(f"fabric constants written to {args.fabric_json}: bws={bws}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
