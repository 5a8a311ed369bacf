#!/usr/bin/env python
"""One LayerNorm (+ residual) forward + backward case for profiling: `python bench/ln_case.py ROWS COLS [iters]`."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from meshslice_b200.ops import functional as F  # noqa: E402

rows, cols = int(sys.argv[1]), int(sys.argv[2])
iters = int(sys.argv[3]) if len(sys.argv) > 3 else 3
x = torch.randn(rows, cols, device="cuda").bfloat16()
res = torch.randn(rows, cols, device="cuda").bfloat16()
g = torch.ones(cols, device="cuda").bfloat16()
b = torch.zeros(cols, device="cuda").bfloat16()
dg = torch.zeros(cols, device="cuda")
db = torch.zeros(cols, device="cuda")
for _ in range(3):  # warm-up; also lets the caching allocator keep the output buffers of two calls
    h, y, mr = F.ln_full(x, res, g, b, 1e-5)
    F.ln_bwd_full(y, h, g, mr, dg, db, res)
ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
ev[0].record()
for _ in range(iters):
    h, y, mr = F.ln_full(x, res, g, b, 1e-5)
ev[1].record()
for _ in range(iters):
    F.ln_bwd_full(y, h, g, mr, dg, db, res)
ev[2].record()
torch.cuda.synchronize()
n = rows * cols * 2
tf, tb = ev[0].elapsed_time(ev[1]) / iters, ev[1].elapsed_time(ev[2]) / iters
print(f"layernorm {rows}x{cols}: fwd {tf * 1e3:.1f} us ({4 * n / tf / 1e6:.0f} GB/s), bwd {tb * 1e3:.1f} us ({4 * n / tb / 1e6:.0f} GB/s)")
