#!/usr/bin/env python
"""One local tcgen05 GEMM case for profiling: `python bench/gemm_case.py M N K layout [iters]`."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from meshslice_b200 import _native  # noqa: E402
from meshslice_b200.ops.gemm import gemm  # noqa: E402

M, N, K = (int(v) for v in sys.argv[1:4])
layout = sys.argv[4] if len(sys.argv) > 4 else "nt"
iters = int(sys.argv[5]) if len(sys.argv) > 5 else 3
a = torch.randn((M, K) if layout != "tn" else (K, M), device="cuda").bfloat16()
b = torch.randn((K, N) if layout != "nt" else (N, K), device="cuda").bfloat16()
out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
gemm(a, b, layout, out=out)
e0.record()
for _ in range(iters):
    gemm(a, b, layout, out=out)
e1.record()
_native.check_status()
ms = e0.elapsed_time(e1) / iters
print(f"{M}x{N}x{K} {layout}: {ms:.4f} ms, {2.0 * M * N * K / ms / 1e9:.1f} TFLOP/s")
