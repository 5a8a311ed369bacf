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


# ----------------------------------------------------------------------------------------------
# timeline of the fused GEMM + collective kernel (events of FusedGemm.read_trace)
# ----------------------------------------------------------------------------------------------
def fused_timeline_summary(events) -> dict:
    """Where the phases of one fused launch lie in time (ns from the first event).

    ``overlap_chunks`` is the share of the gather (first to last ``chunk_sent``) that ran after the first tile
    was complete, ``overlap_sums`` the share of the slot-sum time (``sum_begin`` .. ``sum_end`` per warp) spent
    before the last tile of the launch was complete: both are 0 for a launch that does its phases one after
    another and approach 1 when the transfers hide under the tensor-core work."""
    by = {}
    for e in events:
        by.setdefault(e["kind"], []).append(e)
    span = lambda k: (min(e["t_ns"] for e in by[k]), max(e["t_ns"] for e in by[k])) if k in by else None
    out = {k: dict(first_ns=span(k)[0], last_ns=span(k)[1], count=len(by[k])) for k in by}
    tiles = span("tile_computed")
    chunks = span("chunk_sent")
    if tiles and chunks and chunks[1] > chunks[0]:
        out["overlap_chunks"] = max(0, chunks[1] - max(chunks[0], tiles[0])) / (chunks[1] - chunks[0])
    if tiles and "sum_begin" in by and "sum_end" in by:
        begins = {}
        total = hidden = 0
        for e in sorted(by["sum_begin"] + by["sum_end"], key=lambda e: e["t_ns"]):
            key = (e["cta"], e["arg"])
            if e["kind"] == "sum_begin":
                begins.setdefault(key, []).append(e["t_ns"])
            elif begins.get(key):
                b = begins[key].pop(0)
                total += e["t_ns"] - b
                hidden += max(0, min(e["t_ns"], tiles[1]) - b)
        if total > 0:
            out["overlap_sums"] = hidden / total
    return out


def fused_timeline_to_chrome(events, path: str) -> None:
    """Writes the events as a Chrome trace (one process per CTA; slot sums as spans, the rest as instants)."""
    import json
    recs, open_sums = [], {}
    for e in sorted(events, key=lambda e: e["t_ns"]):
        ts = e["t_ns"] / 1e3
        if e["kind"] == "sum_begin":
            open_sums.setdefault((e["cta"], e["arg"]), []).append(ts)
        elif e["kind"] == "sum_end" and open_sums.get((e["cta"], e["arg"])):
            b = open_sums[(e["cta"], e["arg"])].pop(0)
            recs.append(dict(name=f"slot sums, slice {e['arg']}", ph="X", ts=b, dur=ts - b, pid=e["cta"], tid=1))
        else:
            recs.append(dict(name=f"{e['kind']} {e['arg']}", ph="i", s="t", ts=ts, pid=e["cta"], tid=0))
    with open(path, "w") as f:
        json.dump({"traceEvents": recs, "displayTimeUnit": "ns"}, f)
