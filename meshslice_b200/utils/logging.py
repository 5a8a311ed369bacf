"""Structured run logging: one JSON object per line (config, per-step time, tokens/s, TFLOP/s per
GPU, loss, kernel status) plus a human-readable line on rank 0.  Replaces the bare prints and
shell redirects of the reference (BenchCollectives2D.py:91, runautotune.sh)."""
from __future__ import annotations

import json
import os
import sys
import time
from typing import Optional


class RunLogger:
    def __init__(self, path: Optional[str] = None, rank: int = 0, echo: bool = True):
        self.rank, self.echo = rank, echo and rank == 0
        self.f = open(path, "a") if (path and rank == 0) else None
        self.t0 = time.time()

    def log(self, kind: str, **fields):
        rec = {"t": round(time.time() - self.t0, 3), "kind": kind, **fields}
        if self.f is not None:
            self.f.write(json.dumps(rec) + "\n")
            self.f.flush()
        if self.echo:
            body = " ".join(f"{k}={v:.4g}" if isinstance(v, float) else f"{k}={v}" for k, v in fields.items())
            print(f"[{rec['t']:9.3f}] {kind}: {body}", file=sys.stderr, flush=True)
        return rec

    def close(self):
        if self.f is not None:
            self.f.close()


def read_jsonl(path: str):
    return [json.loads(l) for l in open(path) if l.strip()]
