"""Fused engine of one rank: owns the symmetric heap and workspace and exposes the three
MeshSlice dataflows on local shards, with in-kernel NVLink traffic (no NCCL on these paths).

Gathered operands are pushed: every rank reads its own shard (any device tensor) and writes it
into the peers' staging buffers, so only the workspace lives in the symmetric heap.  When a shape breaks the tile divisibility rules of the fused kernel the
engine falls back to the generic collective formulation (NCCL + local tcgen05 GEMM) and says
so once.
"""
from __future__ import annotations

import warnings
from typing import Optional

import torch

from .. import _native
from ..ops.gemm import gemm, sm_count
from . import runtime as rt
from .fused import FusedGemm, FusedPlanError, MeshCoord
from .mesh import DistMesh, ShardedTensor


def _local(t):
    return t.local() if isinstance(t, ShardedTensor) else t


class FusedEngine:
    def __init__(self, mesh: DistMesh, stage_a_bytes: int, stage_b_bytes: int, slot_bytes: int,
                 extra_heap_bytes: int = 0, timeout_ns: int = 20_000_000_000, exchange_rows: int = 0,
                 allow_fallback: bool = False):
        """``exchange_rows`` > 0 also sets up the in-kernel row exchange among the GPUs of this
        rank's mesh row (LayerNorm statistics, cross-entropy partials) for up to that many rows.
        ``allow_fallback``: a product whose shape breaks the fused kernel's divisibility rules runs
        as NCCL collectives + local GEMM instead of raising (counted in ``fallbacks``)."""
        self.mesh = mesh
        ex_bytes = 2 * mesh.C * exchange_rows * rt.RowExchanger.WIDTH * 4 + 4096 if exchange_rows and mesh.C > 1 else 0
        total = stage_a_bytes + stage_b_bytes + slot_bytes + extra_heap_bytes + ex_bytes + (8 << 20)
        self.heap = rt.SymmHeap(total, group=mesh.group)
        self.ws = rt.Workspace(self.heap, stage_a_bytes, stage_b_bytes, slot_bytes)
        self.world = rt.World.real(self.ws)
        self.coord = MeshCoord(mesh.R, mesh.C, mesh.r, mesh.c)
        self.fg = FusedGemm(self.coord, self.world, sm_count(), timeout_ns=timeout_ns)
        self.row_exchange = None
        if ex_bytes:
            self.row_exchange = rt.RowExchanger(self.heap, self.coord.row_peers(), mesh.c, exchange_rows,
                                                timeout_ns=timeout_ns)
        self.allow_fallback = allow_fallback
        self.fallbacks = 0
        self._warned = set()
        mesh.engine = self

    # ------------------------------------------------------------------ helpers
    @staticmethod
    def _own(t: torch.Tensor, n: int, idx: int):
        """Pointer list indexed by the position along the gathering axis; only this rank's own
        shard is read by its kernel (it is pushed to the peers), so only that entry is set."""
        if t.data_ptr() % 16:
            # every rank must take the same path: copy into an aligned temporary instead of
            # refusing the plan on this rank only
            t = t.clone(memory_format=torch.contiguous_format)
        lst = [0] * n
        lst[idx] = t.data_ptr()
        return lst

    def _fallback(self, which, err, X, W, n_slices):
        if not self.allow_fallback:
            raise FusedPlanError(f"fused {which} not applicable to X {tuple(X.shape)}, W {tuple(W.shape)} on mesh "
                                 f"{self.mesh.R}x{self.mesh.C}: {err} (FusedEngine(allow_fallback=True) runs such "
                                 f"products as NCCL collectives + local GEMM)") from err
        self.fallbacks += 1
        if which not in self._warned:
            warnings.warn(f"fused {which} not applicable ({err}); using NCCL collectives + local GEMM")
            self._warned.add(which)
        from . import tensor_parallel as tp
        m = self.mesh
        Xs = ShardedTensor(m, {(m.r, m.c): X})
        Wsh = ShardedTensor(m, {(m.r, m.c): W})
        fn = {"os": tp.collective_os, "ls": tp.collective_ls, "rs": tp.collective_rs}[which]
        return fn(m, Xs, Wsh).local()

    # ------------------------------------------------------------------ dataflows
    def os(self, X, W, n_slices: int = 4, out: Optional[torch.Tensor] = None, accumulate=False,
           bias=None, act=None, pre_act=None):
        """Y[m, n] = AG_col(X)[m, Kd] @ AG_row(W)[Kd, n]."""
        X, W = _local(X), _local(W)
        m, kl = X.shape
        kr, n = W.shape
        if out is None:
            out = torch.empty(m, n, dtype=torch.bfloat16, device=X.device)
        try:
            X, W = X.contiguous(), W.contiguous()
            xp = self._own(X, self.mesh.C, self.mesh.c)
            wp = self._own(W, self.mesh.R, self.mesh.r)
            return self.fg.os(xp, wp, m, kl, kr, n, out, n_slices=n_slices, accumulate=accumulate,
                              bias=bias, act=act, pre_act=pre_act)
        except FusedPlanError as e:
            y = self._fallback("os", e, X, W, n_slices)
            if bias is not None or act is not None:
                raise
            out.copy_(y) if not accumulate else out.add_(y)
            return out

    def os_kpanel(self, X, W, order: str = "summa", sub: int = 1, out: Optional[torch.Tensor] = None,
                  accumulate=False):
        """The OS product on the K-panel schedule of a baseline algorithm ('summa', 'wang',
        'cannon'): panels of the contraction dimension are pushed by their owners and consumed
        in the order of that algorithm, inside one kernel."""
        X, W = _local(X), _local(W)
        m, kl = X.shape
        kr, n = W.shape
        if out is None:
            out = torch.empty(m, n, dtype=torch.bfloat16, device=X.device)
        try:
            X, W = X.contiguous(), W.contiguous()
            xp = self._own(X, self.mesh.C, self.mesh.c)
            wp = self._own(W, self.mesh.R, self.mesh.r)
            return self.fg.os_kpanel(xp, wp, m, kl, kr, n, out, order=order, sub=sub, accumulate=accumulate)
        except FusedPlanError as e:
            y = self._fallback("os", e, X, W, sub)
            out.copy_(y) if not accumulate else out.add_(y)
            return out

    def ls(self, X, W, n_slices: int = 4, out: Optional[torch.Tensor] = None, accumulate=False, rot_index=None):
        """Y[m, N/C] = RS_col( X[m, kl] @ AG_row(W)[N, kl]^T )."""
        X, W = _local(X), _local(W)
        m, kl = X.shape
        nr = W.shape[0]
        N = nr * self.mesh.R
        if out is None:
            out = torch.empty(m, N // self.mesh.C, dtype=torch.bfloat16, device=X.device)
        try:
            W = W.contiguous()
            wp = self._own(W, self.mesh.R, self.mesh.r)
            return self.fg.ls(X.contiguous(), wp, m, kl, nr, out, n_slices=n_slices, accumulate=accumulate,
                              rot_index=rot_index)
        except FusedPlanError as e:
            y = self._fallback("ls", e, X, W, n_slices)
            out.copy_(y) if not accumulate else out.add_(y)
            return out

    def rs(self, X, W, n_slices: int = 4, out: Optional[torch.Tensor] = None, accumulate=False, rot_index=None):
        """Y[M/R, n] = RS_row( AG_col(X)[kr, M]^T @ W[kr, n] )."""
        X, W = _local(X), _local(W)
        kr, ml = X.shape
        n = W.shape[1]
        M = ml * self.mesh.C
        if out is None:
            out = torch.empty(M // self.mesh.R, n, dtype=torch.bfloat16, device=X.device)
        try:
            X = X.contiguous()
            xp = self._own(X, self.mesh.C, self.mesh.c)
            return self.fg.rs(xp, W.contiguous(), kr, ml, n, out, n_slices=n_slices, accumulate=accumulate,
                              rot_index=rot_index)
        except FusedPlanError as e:
            y = self._fallback("rs", e, X, W, n_slices)
            out.copy_(y) if not accumulate else out.add_(y)
            return out

    def check(self):
        """Raise if any kernel of this process reported a timeout (synchronises the device)."""
        _native.check_status()


class LocalGemmEngine:
    """Engine of a 1 x 1 mesh: the three dataflows degenerate to local tcgen05 GEMMs in the
    'nn' / 'nt' / 'tn' layouts (no operand is transposed in memory)."""

    def __init__(self, mesh):
        self.mesh = mesh
        mesh.engine = self

    @staticmethod
    def _run(X, W, layout, out, accumulate, **kw):
        X, W = _local(X), _local(W)
        return gemm(X, W, layout, out=out, accumulate=accumulate, **kw)

    def os(self, X, W, n_slices=1, out=None, accumulate=False, bias=None, act=None, pre_act=None):
        return self._run(X, W, "nn", out, accumulate, bias=bias, act=act, pre_act=pre_act)

    def os_kpanel(self, X, W, order="summa", sub=1, out=None, accumulate=False):
        return self._run(X, W, "nn", out, accumulate)

    def ls(self, X, W, n_slices=1, out=None, accumulate=False, rot_index=None):
        return self._run(X, W, "nt", out, accumulate)

    def rs(self, X, W, n_slices=1, out=None, accumulate=False, rot_index=None):
        return self._run(X, W, "tn", out, accumulate)

    def check(self):
        _native.check_status()
