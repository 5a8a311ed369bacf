#!/usr/bin/env python
"""Local tcgen05 GEMM against torch.matmul (cuBLAS) on the per-device shapes of the GPT-3 6.7B training step.

`python bench/BenchGemmLocal.py [--reps 10] [--knobs]`

Every shape runs all arms round-robin inside each repetition, so that the clock drift of a power-capped GPU hits
every arm alike; L2 is flushed (a 256 MiB write) before each timed call; times are CUDA-event medians.  With
`--knobs` the kernel's stage count (6 / 7) and the 3-D tensor map of MN-major operands (off / on) are swept as
separate arms through the environment variables that `meshslice_b200.ops.gemm.gemm` reads.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from meshslice_b200 import _native  # noqa: E402
from meshslice_b200.ops.gemm import gemm  # noqa: E402

SHAPES = [(8192, 8192, 8192, "nt"), (8192, 12288, 4096, "nn"), (8192, 16384, 4096, "nn"), (8192, 4096, 16384, "nt"),
          (8192, 4096, 4096, "nn"), (4096, 16384, 8192, "tn"), (8192, 51200, 4096, "nn"), (8192, 4096, 12288, "nt"),
          (4096, 12288, 8192, "tn"), (16384, 4096, 8192, "tn")]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--knobs", action="store_true")
    args = ap.parse_args()
    arms = [("cublas", None)]
    if args.knobs:
        arms += [(f"s{st}m{m3}", dict(MSB_G2_STAGES=str(st), MSB_G2_MAP3D=str(m3))) for st in (6, 7) for m3 in (0, 1)]
    else:
        arms += [("gemm", {})]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    total = {name: 0.0 for name, _ in arms}
    for (M, N, K, lay) in SHAPES:
        a = torch.randn((M, K) if lay != "tn" else (K, M), device="cuda").bfloat16()
        b = torch.randn((K, N) if lay != "nt" else (N, K), device="cuda").bfloat16()
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        lhs = a.t() if lay == "tn" else a
        rhs = b.t() if lay == "nt" else b
        times = {name: [] for name, _ in arms}
        for rep in range(args.reps + 2):
            for name, env in arms:
                if env:
                    os.environ.update(env)
                flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                if env is None:
                    torch.matmul(lhs, rhs, out=out)
                else:
                    gemm(a, b, lay, out=out)
                e1.record()
                torch.cuda.synchronize()
                if rep >= 2:
                    times[name].append(e0.elapsed_time(e1))
        _native.check_status()
        gflop = 2.0 * M * N * K / 1e9
        line = f"{M}x{N}x{K} {lay}: "
        for name, _ in arms:
            t = sorted(times[name])[len(times[name]) // 2]
            total[name] += t
            line += f"{name} {gflop / t:6.0f}  "
        print(line, flush=True)
    print("total ms: " + "  ".join(f"{k} {v:.3f}" for k, v in total.items()))


if __name__ == "__main__":
    main()
