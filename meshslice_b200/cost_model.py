"""Analytical cost model of the 2-D GeMM algorithms (counterpart of CostModel.py).

Same public names and return conventions as the reference: every algorithm model returns
``(prologue, steady_state)`` in seconds, where the prologue is communication that cannot be
overlapped.  Differences, all deliberate:

* ``estimateMatmul`` is pluggable.  The reference always *measures* a jitted einsum on the local
  chip (CostModel.py:74-98); here a ``MatmulEstimator`` is either analytic (peak FLOP/s with an
  efficiency curve, works without a GPU), a lookup table, or measured with the tcgen05 GEMM.
* Fabric models.  ``fabric='ring'`` keeps the reference's torus formulas
  ``base + (n-1) * bytes / bw + (n-1) * latency`` (CostModel.py:47-63).  ``fabric='switch'`` models
  NVLink 5 through NVSwitch: every peer is one hop away, an all-gather moves ``(n-1) * bytes`` into
  each GPU's single port at the port bandwidth, latency does not grow with n, and collectives on
  the row and column axes share that port (``shared_port=True`` adds their times where the torus
  model takes the maximum, cf. CostModel.py:258).
* The reference's broken paths are fixed: ``estimateBroadcast`` used ``bw`` before assigning it
  (CostModel.py:35-38) and the Cannon models called ``estimateSkew`` without its precision
  argument (CostModel.py:176-211).
"""
from __future__ import annotations

import json
import math
import time
from dataclasses import dataclass, field
from typing import Dict, Optional, Tuple

Shape2 = Tuple[int, int]


# ----------------------------------------------------------------------------------------------
# matmul time
# ----------------------------------------------------------------------------------------------
class MatmulEstimator:
    """Time of one local GEMM [M,K] x [K,N] in seconds."""

    def __call__(self, M: int, N: int, K: int, layout: str = "nn") -> float:
        raise NotImplementedError


class AnalyticMatmul(MatmulEstimator):
    """peak * efficiency(size): small GEMMs are launch/tail bound, large ones reach ``eff``."""

    def __init__(self, peak_flops: float = 1.38e15, eff: float = 0.85, launch: float = 6e-6, n_sm: int = 148,
                 tile=(128, 256)):
        self.peak, self.eff, self.launch, self.n_sm, self.tile = peak_flops, eff, launch, n_sm, tile

    def __call__(self, M, N, K, layout="nn"):
        tm, tn = self.tile
        tiles = math.ceil(M / tm) * math.ceil(N / tn)
        waves = math.ceil(tiles / self.n_sm)
        per_tile = 2.0 * tm * tn * K / (self.peak * self.eff / self.n_sm)
        return self.launch + waves * per_tile


class TableMatmul(MatmulEstimator):
    """Measured times keyed by (M, N, K, layout); falls back to another estimator."""

    def __init__(self, table: Dict[str, float], fallback: Optional[MatmulEstimator] = None):
        self.table, self.fallback = table, fallback or AnalyticMatmul()

    def __call__(self, M, N, K, layout="nn"):
        key = f"{M},{N},{K},{layout}"
        return self.table[key] if key in self.table else self.fallback(M, N, K, layout)


class MeasuredMatmul(MatmulEstimator):
    """Times the tcgen05 GEMM of this package on the current GPU (CUDA events, bf16)."""

    def __init__(self, repeat: int = 5, max_bytes: int = 8 << 30):
        self.repeat, self.cache, self.max_bytes = repeat, {}, max_bytes

    def __call__(self, M, N, K, layout="nn"):
        key = (M, N, K, layout)
        if key in self.cache:
            return self.cache[key]
        import torch
        from .ops.gemm import gemm
        if 2 * (M * K + K * N + M * N) > self.max_bytes:
            raise MemoryError("matmul probe larger than the configured bound")
        a = torch.ones((M, K) if layout != "tn" else (K, M), dtype=torch.bfloat16, device="cuda")
        b = torch.ones((K, N) if layout != "nt" else (N, K), dtype=torch.bfloat16, device="cuda")
        out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        gemm(a, b, layout, out=out)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(self.repeat):
            gemm(a, b, layout, out=out)
        e1.record()
        torch.cuda.synchronize()
        t = e0.elapsed_time(e1) * 1e-3 / self.repeat
        self.cache[key] = t
        return t


_default_matmul: MatmulEstimator = AnalyticMatmul()


def set_default_matmul(est: MatmulEstimator) -> None:
    global _default_matmul
    _default_matmul = est


# ----------------------------------------------------------------------------------------------
# mesh description
# ----------------------------------------------------------------------------------------------
class DeviceMesh:
    """Mesh shape plus fabric constants (CostModel.py:8-29).

    ``bws_per_direction[kind]`` is a pair (bandwidth along mesh dim 0, along mesh dim 1) in bytes/s
    for kind in {'allgather', 'reducescatter', 'sendrecv'}; ``link_latencies`` and ``base_overheads``
    are per kind in seconds.  A tuple entry in ``device_shape`` folds a 2-D sub-mesh into one
    logical dimension (hierarchical dimension, CostModel.py:16-29)."""

    def __init__(self, device_shape: tuple, flops_per_chip: float, bws_per_direction, link_latencies,
                 base_overheads, fabric: str = "ring", shared_port: bool = False,
                 matmul: Optional[MatmulEstimator] = None, fused: Optional["FusedKernelConstants"] = None):
        self.reshape(device_shape)
        self.fused = fused
        self.flops = flops_per_chip
        self.bws = bws_per_direction
        self.link_latencies = link_latencies
        self.base_overheads = base_overheads
        self.fabric = fabric
        self.shared_port = shared_port
        self.matmul = matmul

    def reshape(self, newshape):
        self.meshdim = None
        self.submesh = None
        if isinstance(newshape[0], tuple):
            self.meshdim, self.submesh = 0, newshape[0]
            self.shape = (newshape[0][0] * newshape[0][1], newshape[1])
        elif isinstance(newshape[1], tuple):
            self.meshdim, self.submesh = 1, newshape[1]
            self.shape = (newshape[0], newshape[1][0] * newshape[1][1])
        else:
            self.shape = tuple(newshape)

    def combine(self, *times: float) -> float:
        """Concurrent collectives on different mesh axes: disjoint links on a torus (max), one
        shared NVLink port per GPU behind a switch (sum)."""
        return sum(times) if self.shared_port else max(times)

    @classmethod
    def from_fabric_json(cls, device_shape, path_or_dict, **kw):
        """Builds a mesh from the constants fitted by BenchCollectives2D (``--fabric-json``)."""
        d = path_or_dict if isinstance(path_or_dict, dict) else json.load(open(path_or_dict))
        bws = {k: tuple(v) if isinstance(v, (list, tuple)) else (v, v) for k, v in d["bws"].items()}
        if "fused" in d and "fused" not in kw:
            kw["fused"] = FusedKernelConstants(**d["fused"])
        return cls(device_shape, d.get("flops_per_chip", 1.38e15), bws, d["latencies"], d["base_overheads"],
                   fabric=d.get("fabric", "switch"), shared_port=d.get("shared_port", True), **kw)


def bytesize(shape: Shape2) -> int:
    return shape[0] * shape[1] * 2


def _size(shape: Shape2, precision: int) -> float:
    return shape[0] * shape[1] * precision // 8


def _hier(mesh, dim, data_size, bw, link_latency, base_overhead, full: bool):
    r, c = mesh.submesh
    half = data_size // 2
    if full:
        total_latency = link_latency * (r + c - 2)
        row_first = (half / bw) * (r - 1) + (half * r / bw) * (c - 1)
        col_first = (half / bw) * (c - 1) + (half * c / bw) * (r - 1)
        return base_overhead + max(row_first, col_first) + total_latency
    return base_overhead + half / bw + link_latency * (r + c - 1)


def _gather_like(mesh: DeviceMesh, kind: str, data_shape: Shape2, dim: int, precision: int) -> float:
    data_size = _size(data_shape, precision)
    n = mesh.shape[dim]
    steps = n - 1
    lat, base, bw = mesh.link_latencies[kind], mesh.base_overheads[kind], mesh.bws[kind][dim]
    if steps == 0:
        return 0.0
    if dim == mesh.meshdim:
        return _hier(mesh, dim, data_size, bw, lat, base, full=True)
    if mesh.fabric == "switch":
        return base + lat + steps * data_size / bw
    return base + steps * data_size / bw + lat * steps


def estimateAllgather(mesh: DeviceMesh, data_shape: Shape2, dim: int, precision: int = 16) -> float:
    """All-gather of per-device shards ``data_shape`` among the devices along mesh dim ``dim``."""
    return _gather_like(mesh, "allgather", data_shape, dim, precision)


def estimateReduceScatter(mesh: DeviceMesh, data_shape: Shape2, dim: int, precision: int = 16) -> float:
    """Reduce-scatter whose per-device result has shape ``data_shape``."""
    return _gather_like(mesh, "reducescatter", data_shape, dim, precision)


def _one_to_all(mesh, kind, data_shape, dim, precision):
    data_size = _size(data_shape, precision)
    lat, base, bw = mesh.link_latencies[kind], mesh.base_overheads[kind], mesh.bws[kind][dim]
    n = mesh.shape[dim]
    if n == 1:
        return 0.0
    if dim == mesh.meshdim:
        return _hier(mesh, dim, data_size, bw, lat, base, full=False)
    if mesh.fabric == "switch":
        # one source port feeds n-1 peers unless the switch replicates (multimem): bounded by egress
        return base + lat + (n - 1) * data_size / bw
    return base + data_size / bw + lat * (n - 1)


def estimateBroadcast(mesh, data_shape, dim, precision=16):
    """Pipelined broadcast (SUMMA panels)."""
    return _one_to_all(mesh, "allgather", data_shape, dim, precision)


def estimateReduce(mesh, data_shape, dim, precision=16):
    return _one_to_all(mesh, "reducescatter", data_shape, dim, precision)


def estimateSkew(mesh, data_shape, precision=16):
    """Initial alignment of Cannon's algorithm: shift by up to half the (square) mesh."""
    assert mesh.shape[0] == mesh.shape[1]
    lat, base, bw = mesh.link_latencies["sendrecv"], mesh.base_overheads["sendrecv"], mesh.bws["sendrecv"][1]
    steps = 1 if mesh.fabric == "switch" else mesh.shape[0] // 2
    return base + steps * _size(data_shape, precision) / bw + lat * steps


def estimateMatmul(mesh, M, N, K, input_precision=None, layout="nn", repeat=5) -> float:
    est = mesh.matmul if mesh is not None and getattr(mesh, "matmul", None) is not None else _default_matmul
    return est(int(M), int(N), int(K), layout)


# ----------------------------------------------------------------------------------------------
# algorithm models
# ----------------------------------------------------------------------------------------------
def SUMMA_OS(mesh, M, N, K, steps=8, precisions=(16, 16, 16)):
    steps = math.lcm(mesh.shape[0], mesh.shape[1])
    ishape = (M // mesh.shape[0], K // steps)
    wshape = (K // steps, N // mesh.shape[1])
    bi = estimateBroadcast(mesh, ishape, 1, precisions[0])
    bw_ = estimateBroadcast(mesh, wshape, 0, precisions[1])
    comm = mesh.combine(bi, bw_)
    compute = estimateMatmul(mesh, ishape[0], wshape[1], ishape[1])
    return (comm, max(comm, compute) * (steps - 1) + compute)


def SUMMA_LS(mesh, M, N, K, steps=8, precisions=(16, 16, 16)):
    steps = math.lcm(mesh.shape[0], mesh.shape[1])
    ishape = (M // mesh.shape[0], K // mesh.shape[1])
    oshape = (M // mesh.shape[0], N // steps)
    wshape = (N // steps, K // mesh.shape[1])
    b = estimateBroadcast(mesh, wshape, 0, precisions[1])
    r = estimateReduce(mesh, oshape, 1, precisions[2])
    compute = estimateMatmul(mesh, ishape[0], oshape[1], ishape[1], layout="nt")
    return (b + r, max(mesh.combine(r, b), compute) * (steps - 1) + compute)


def SUMMA_RS(mesh, M, N, K, steps=8, precisions=(16, 16, 16)):
    steps = math.lcm(mesh.shape[0], mesh.shape[1])
    ishape = (K // mesh.shape[0], M // steps)
    oshape = (M // steps, N // mesh.shape[1])
    wshape = (K // mesh.shape[0], N // mesh.shape[1])
    b = estimateBroadcast(mesh, ishape, 1, precisions[0])
    r = estimateReduce(mesh, oshape, 0, precisions[2])
    compute = estimateMatmul(mesh, oshape[0], oshape[1], wshape[0], layout="tn")
    return (b + r, max(mesh.combine(r, b), compute) * (steps - 1) + compute)


def _roll(mesh, shape):
    lat, base, bw = mesh.link_latencies["sendrecv"], mesh.base_overheads["sendrecv"], mesh.bws["sendrecv"][1]
    return bytesize(shape) / bw + lat + base


def Cannon_OS(mesh, M, N, K, steps=8, precisions=(16, 16, 16)):
    ishape = (M // mesh.shape[0], K // mesh.shape[1])
    wshape = (K // mesh.shape[0], N // mesh.shape[1])
    skew = max(estimateSkew(mesh, ishape, precisions[0]), estimateSkew(mesh, wshape, precisions[1]))
    compute = estimateMatmul(mesh, ishape[0], wshape[1], ishape[1])
    roll = mesh.combine(_roll(mesh, ishape), _roll(mesh, wshape))
    return (skew, mesh.shape[0] * max(roll, compute))


def Cannon_LS(mesh, M, N, K, steps=8, precisions=(16, 16, 16)):
    ishape = (M // mesh.shape[0], K // mesh.shape[1])
    wshape = (N // mesh.shape[0], K // mesh.shape[1])
    oshape = (M // mesh.shape[0], N // mesh.shape[1])
    skew = max(estimateSkew(mesh, oshape, precisions[2]), estimateSkew(mesh, wshape, precisions[1]))
    compute = estimateMatmul(mesh, oshape[0], oshape[1], ishape[1], layout="nt")
    roll = mesh.combine(_roll(mesh, oshape), _roll(mesh, wshape))
    return (skew, mesh.shape[0] * max(roll, compute))


def Cannon_RS(mesh, M, N, K, steps=8, precisions=(16, 16, 16)):
    ishape = (K // mesh.shape[0], M // mesh.shape[1])
    oshape = (M // mesh.shape[0], N // mesh.shape[1])
    skew = max(estimateSkew(mesh, oshape, precisions[2]), estimateSkew(mesh, ishape, precisions[0]))
    compute = estimateMatmul(mesh, oshape[0], oshape[1], ishape[0], layout="tn")
    roll = mesh.combine(_roll(mesh, oshape), _roll(mesh, ishape))
    return (skew, mesh.shape[0] * max(roll, compute))


def GSPMD_OS(mesh, M, N, K, steps=8, precisions=(16, 16, 16)):
    ishape = (M // mesh.shape[0], K // mesh.shape[1])
    wshape = (K // mesh.shape[0], N // mesh.shape[1])
    ag_i = estimateAllgather(mesh, ishape, 1, precisions[0])
    ag_w = estimateAllgather(mesh, wshape, 0, precisions[1])
    compute = estimateMatmul(mesh, ishape[0], wshape[1], K)
    return (ag_i, max(compute, ag_w)) if not mesh.shared_port else (ag_i + ag_w, compute)


def GSPMD_LS(mesh, M, N, K, steps=8, precisions=(16, 16, 16)):
    ishape = (M // mesh.shape[0], K // mesh.shape[1])
    wshape = (N // mesh.shape[0], K // mesh.shape[1])
    oshape = (M // mesh.shape[0], N // mesh.shape[1])
    ag_w = estimateAllgather(mesh, wshape, 0, precisions[1])
    compute = estimateMatmul(mesh, ishape[0], N, ishape[1], layout="nt")
    rs_o = estimateReduceScatter(mesh, oshape, 1, precisions[2])
    return (rs_o, max(ag_w, compute)) if not mesh.shared_port else (rs_o + ag_w, compute)


def GSPMD_RS(mesh, M, N, K, steps=8, precisions=(16, 16, 16)):
    ishape = (K // mesh.shape[0], M // mesh.shape[1])
    wshape = (K // mesh.shape[0], N // mesh.shape[1])
    oshape = (M // mesh.shape[0], N // mesh.shape[1])
    ag_i = estimateAllgather(mesh, ishape, 1, precisions[0])
    compute = estimateMatmul(mesh, M, wshape[1], ishape[0], layout="tn")
    rs_o = estimateReduceScatter(mesh, oshape, 0, precisions[2])
    return (rs_o, max(ag_i, compute)) if not mesh.shared_port else (rs_o + ag_i, compute)


def MeshFlow_OS(mesh, M, N, K, steps=32, precisions=(16, 16, 16)):
    """Sliced OS: prologue = first slice's gathers, then max(comm, compute) per remaining slice."""
    ishape = (M // mesh.shape[0], K // mesh.shape[1] // steps)
    wshape = (K // mesh.shape[0] // steps, N // mesh.shape[1])
    ag_i = estimateAllgather(mesh, ishape, 1, precisions[0])
    ag_w = estimateAllgather(mesh, wshape, 0, precisions[1])
    comm = mesh.combine(ag_i, ag_w)
    compute = estimateMatmul(mesh, ishape[0], wshape[1], K) / steps
    return (comm, max(comm, compute) * (steps - 1) + compute)


def MeshFlow_LS(mesh, M, N, K, steps=32, precisions=(16, 16, 16)):
    ishape = (M // mesh.shape[0], K // mesh.shape[1])
    wshape = (N // mesh.shape[0] // steps, K // mesh.shape[1])
    oshape = (M // mesh.shape[0], N // mesh.shape[1] // steps)
    ag_w = estimateAllgather(mesh, wshape, 0, precisions[1])
    rs_o = estimateReduceScatter(mesh, oshape, 1, precisions[2])
    compute = estimateMatmul(mesh, ishape[0], N, ishape[1], layout="nt") / steps
    return (ag_w + rs_o, compute + max(mesh.combine(ag_w, rs_o), compute) * (steps - 1))


def MeshFlow_RS(mesh, M, N, K, steps=32, precisions=(16, 16, 16)):
    ishape = (K // mesh.shape[0], M // mesh.shape[1] // steps)
    wshape = (K // mesh.shape[0], N // mesh.shape[1])
    oshape = (M // mesh.shape[0] // steps, N // mesh.shape[1])
    ag_i = estimateAllgather(mesh, ishape, 1, precisions[0])
    rs_o = estimateReduceScatter(mesh, oshape, 0, precisions[2])
    compute = estimateMatmul(mesh, M, oshape[1], ishape[0], layout="tn") / steps
    return (ag_i + rs_o, compute + max(mesh.combine(ag_i, rs_o), compute) * (steps - 1))


# ----------------------------------------------------------------------------------------------
# models of the fused tcgen05 GEMM + collective kernel (csrc/gemm/sm100_gemm.cu), i.e. of what runs on GPUs
# ----------------------------------------------------------------------------------------------
@dataclass
class FusedKernelConstants:
    """Rates of the fused kernel, fitted from `bench/BenchGemm2D.py` sweeps by `bench/fit_fused_model.py`.

    The MeshFlow_* models above keep the reference's view (every slice is a collective followed by a
    GEMM, CostModel.py:214-262).  The kernel that runs differs in four ways that matter for time: one launch
    per product with a cross-GPU entry and exit barrier; shards are *pushed* by the SMs that also compute, so
    a gather is faster before the first tile than under tiles; partial tiles are pushed to their owners from
    the epilogue; the owners' slot sums run beside the tiles and only the last slice's sum is exposed."""
    launch_overhead: float = 1.0e-4      # s per launch: barriers across GPUs, first-chunk latency, tail
    gather_bw_alone: float = 560e9       # bytes/s a GPU pushes while none of its tiles run
    gather_bw_overlap: float = 300e9     # ... while tiles run on the same SMs
    push_bw: float = 450e9               # bytes/s of partial tiles pushed from the epilogue
    slot_sum_bw: float = 2.2e12          # bytes/s of slot reads in the per-slice sums
    tile_eff: float = 0.93               # main-loop rate relative to the matmul estimator
    slice_overhead: float = 0.0          # s per slice: flag waits, fences and counter updates at slice boundaries
    matmul_peak: float = 1.3806e15       # FLOP/s of the analytic estimator that tile_eff was fitted against

    def to_dict(self):
        return dict(self.__dict__)


def _fused(mesh) -> FusedKernelConstants:
    f = getattr(mesh, "fused", None)
    return f if f is not None else FusedKernelConstants()


def _tiles(mesh, M, N, K, layout):
    f = _fused(mesh)
    if getattr(mesh, "matmul", None) is not None:          # measured or tabulated GEMM times
        return mesh.matmul(int(M), int(N), int(K), layout) / f.tile_eff
    return AnalyticMatmul(peak_flops=f.matmul_peak, eff=1.0)(int(M), int(N), int(K), layout) / f.tile_eff


def Fused_OS(mesh, M, N, K, steps=4, precisions=(16, 16, 16)):
    """Y[M/R, N/C] = gather_cols(X[M/R, K/C]) . gather_rows(W[K/R, N/C]): X travels as `steps` row slices, W as
    column chunks, interleaved in order of first use; the first tile needs one piece of each."""
    R, C = mesh.shape
    f = _fused(mesh)
    bx = (C - 1) * _size((M // R, K // C), precisions[0])
    bw = (R - 1) * _size((K // R, N // C), precisions[1])
    tiles = _tiles(mesh, M // R, N // C, K, "nn")
    if bx + bw == 0:
        return (0.0, tiles)
    first = (bx + bw) / steps / f.gather_bw_alone
    rest = (bx + bw) * (1.0 - 1.0 / steps) / f.gather_bw_overlap
    return (f.launch_overhead + first, max(tiles, rest) + steps * f.slice_overhead)


def _fused_scatter(mesh, gather_bytes, push_bytes, slot_bytes, tiles, steps):
    f = _fused(mesh)
    if gather_bytes + push_bytes == 0:
        return (0.0, tiles)
    first = gather_bytes / steps / f.gather_bw_alone
    under = gather_bytes * (1.0 - 1.0 / steps) / f.gather_bw_overlap + push_bytes / f.push_bw
    tail = slot_bytes / steps / f.slot_sum_bw      # the last slice's slot sum has no tiles left to hide under
    return (f.launch_overhead + first, max(tiles, under) + tail + steps * f.slice_overhead)


def Fused_LS(mesh, M, N, K, steps=4, precisions=(16, 16, 16)):
    """Y[M/R, N/C] = scatter_cols(X[M/R, K/C] . gather_rows(W[N/R, K/C])^T): output columns are sliced."""
    R, C = mesh.shape
    bw = (R - 1) * _size((N // R, K // C), precisions[1])
    part = _size((M // R, N), precisions[2])
    push = part * (C - 1) / C
    slots = part if C > 1 else 0.0
    return _fused_scatter(mesh, bw, push, slots, _tiles(mesh, M // R, N, K // C, "nt"), steps)


def Fused_RS(mesh, M, N, K, steps=4, precisions=(16, 16, 16)):
    """Y[M/R, N/C] = scatter_rows(gather_cols(X[K/R, M/C])^T . W[K/R, N/C]): output rows are sliced."""
    R, C = mesh.shape
    bx = (C - 1) * _size((K // R, M // C), precisions[0])
    part = _size((M, N // C), precisions[2])
    push = part * (R - 1) / R
    slots = part if R > 1 else 0.0
    return _fused_scatter(mesh, bx, push, slots, _tiles(mesh, M, N // C, K // R, "tn"), steps)


def _ring(mesh, shape, M_, N_, K_):
    P = mesh.shape[0] * mesh.shape[1]
    lat, base, bw = mesh.link_latencies["sendrecv"], mesh.base_overheads["sendrecv"], mesh.bws["sendrecv"][1]
    roll = bytesize(shape) / (bw * 2) + lat + base
    return (0, max(roll, estimateMatmul(mesh, M_, N_, K_)) * P)


def LogicalRing_ISplit(mesh, M, N, K, steps=8):
    P = mesh.shape[0] * mesh.shape[1]
    return _ring(mesh, (M, K // P), M, N // P, K // P)


def LogicalRing_WSplit(mesh, M, N, K, steps=8):
    P = mesh.shape[0] * mesh.shape[1]
    return _ring(mesh, (K // P, N), M // P, N, K // P)


def LogicalRing_OSplit(mesh, M, N, K, steps=8):
    P = mesh.shape[0] * mesh.shape[1]
    return _ring(mesh, (M, N // P), M, N // P, K // P)


def tup2ms(t):
    return (str(t[0] * 1000) + "ms", str(t[1] * 1000) + "ms", str((t[0] + t[1]) * 1000) + "ms")
