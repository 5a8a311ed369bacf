"""Device-side timing and trace annotations.

``DeviceTimer`` brackets a region with CUDA events on the current stream and reports the maximum
over ranks, the way every multi-GPU number of this package is taken.  ``annotate`` opens an NVTX
range (visible in Nsight / torch.profiler traces) with the reference's tags, replacing
jax.profiler.TraceAnnotation (BenchTransformer.py:105-110).  ``trace`` writes a Chrome trace with
torch.profiler instead of a TensorBoard directory.
"""
from __future__ import annotations

import contextlib
from typing import Optional

import torch


class DeviceTimer:
    def __init__(self, group=None):
        self.group = group
        self.e0 = torch.cuda.Event(enable_timing=True)
        self.e1 = torch.cuda.Event(enable_timing=True)

    def __enter__(self):
        torch.cuda.synchronize()
        self.e0.record()
        return self

    def __exit__(self, *exc):
        self.e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([self.e0.elapsed_time(self.e1)], device="cuda")
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(self.group) > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX, group=self.group)
        self.ms = ms.item()
        return False


@contextlib.contextmanager
def annotate(tag: str):
    """NVTX range; a no-op without CUDA."""
    use = torch.cuda.is_available()
    if use:
        torch.cuda.nvtx.range_push(tag)
    try:
        yield
    finally:
        if use:
            torch.cuda.nvtx.range_pop()


@contextlib.contextmanager
def trace(path: Optional[str]):
    """Chrome-trace export of the enclosed region (rank-local file)."""
    if not path:
        yield None
        return
    from torch.profiler import ProfilerActivity, profile
    acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
    with profile(activities=acts) as prof:
        yield prof
    prof.export_chrome_trace(path)
