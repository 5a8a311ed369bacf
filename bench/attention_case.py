#!/usr/bin/env python
"""One attention forward + backward case for profiling:
`python bench/attention_case.py BATCH SEQ HEADS [causal] [iters]` (head_dim 128)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from meshslice_b200 import _native  # noqa: E402
from meshslice_b200.ops import functional as F  # noqa: E402

batch, seq, heads = (int(v) for v in sys.argv[1:4])
causal = (sys.argv[4] if len(sys.argv) > 4 else "1") != "0"
iters = int(sys.argv[5]) if len(sys.argv) > 5 else 3
qkv = torch.randn(batch * seq, heads * 3 * 128, device="cuda").bfloat16()
dout = torch.randn(batch * seq, heads * 128, device="cuda").bfloat16()
out, lse = F.attention_fwd(qkv, batch, seq, heads, causal)
F.attention_bwd(dout, qkv, out, lse, batch, seq, heads, causal)
ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
ev[0].record()
for _ in range(iters):
    out, lse = F.attention_fwd(qkv, batch, seq, heads, causal)
ev[1].record()
for _ in range(iters):
    F.attention_bwd(dout, qkv, out, lse, batch, seq, heads, causal)
ev[2].record()
_native.check_status()
f = 4.0 * batch * heads * seq * seq * 128 * (0.5 if causal else 1.0)
tf, tb = ev[0].elapsed_time(ev[1]) / iters, ev[1].elapsed_time(ev[2]) / iters
print(f"attention b{batch} s{seq} h{heads} causal={causal}: fwd {tf:.3f} ms ({f / tf / 1e9:.0f} TFLOP/s), "
      f"bwd {tb:.3f} ms ({2.5 * f / tb / 1e9:.0f} TFLOP/s)")
