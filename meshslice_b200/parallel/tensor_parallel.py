"""2-D tensor-parallel GeMM algorithms and the ``SPMD`` builder.

Public surface mirrors the reference (TensorParallel.py:346-377): ``SPMD(mesh, algorithm,
blocksize).OS(K) / .LS(K) / .RS(K)`` return callables on block-sharded operands
(``ShardedTensor``, P(row, col)) that compute

    OS:  Y = X  @ W      X [M, Kd],  W [Kd, N]
    LS:  Y = X  @ W^T    X [M, Kd],  W [N, Kd]
    RS:  Y = X^T @ W     X [Kd, M],  W [Kd, N]

with Y block-sharded the same way.  Algorithms: 'meshslice' (alias 'meshflow', the product:
sliced all-gather / reduce-scatter, TensorParallel.py:153-214), 'collective' (monolithic
collectives, :19-32), 'wang' (bidirectional ring collective-matmul, :34-149), 'cannon' (square
meshes, :218-344 and :379-417) and 'summa' (broadcast/reduce panels; the reference only has a
cost model for it, CostModel.py:136-168).

Every algorithm here is written once against the ``Mesh`` interface, so the same code is the
CPU oracle (EmuMesh), the Gloo multi-process path and the NCCL + library-GEMM baseline
(DistMesh).  On a GPU DistMesh, 'meshslice' dispatches to the fused tcgen05 kernels of
``parallel.fused`` instead (see ``parallel.engine``).
"""
from __future__ import annotations

import math
from functools import partial
from typing import Callable

import torch

from .mesh import DistMesh, EmuMesh, Mesh, ShardedTensor


def allclose(a, b, atol=1e-2, rtol=1e-2) -> bool:
    """Tolerance of the reference's self-tests (TensorParallel.py:16-17)."""
    if isinstance(a, ShardedTensor):
        return all(torch.allclose(a.shards[k].float(), b.shards[k].float(), atol=atol, rtol=rtol)
                   for k in a.shards)
    return torch.allclose(a.float(), b.float(), atol=atol, rtol=rtol)


def _mm(a, b):
    """Local product with fp32 accumulation (bf16 inputs use the library GEMM on GPUs)."""
    if a.dtype in (torch.bfloat16, torch.float16) and a.device.type == "cpu":
        return (a.float() @ b.float()).to(a.dtype)
    return a @ b


# ----------------------------------------------------------------------------------------------
# collective (GSPMD-style) baseline
# ----------------------------------------------------------------------------------------------
def collective_os(mesh: Mesh, X, W, K=1, B=8):
    Xi = mesh.all_gather(X, "col", 1)
    Wj = mesh.all_gather(W, "row", 0)
    return mesh.map(lambda r, c, x, w: _mm(x, w), Xi, Wj)


def collective_ls(mesh: Mesh, X, W, K=1, B=8):
    Wj = mesh.all_gather(W, "row", 0)
    Yp = mesh.map(lambda r, c, x, w: _mm(x, w.t()), X, Wj)
    return mesh.reduce_scatter(Yp, "col", 1)


def collective_rs(mesh: Mesh, X, W, K=1, B=8):
    Xi = mesh.all_gather(X, "col", 1)
    Yp = mesh.map(lambda r, c, x, w: _mm(x.t(), w), Xi, W)
    return mesh.reduce_scatter(Yp, "row", 0)


# ----------------------------------------------------------------------------------------------
# MeshSlice: block-cyclic slices of the moving dimension
# ----------------------------------------------------------------------------------------------
def slice_indices(length: int, K: int, B: int, i: int) -> torch.Tensor:
    """Local indices of slice i: { k : (k // B) mod K == i } (TensorParallel.py:155-158)."""
    if length % (K * B):
        raise ValueError(f"length {length} is not a multiple of slices*block = {K}*{B}")
    k = torch.arange(length)
    return k[(k // B) % K == i]


def _check_div(length, K, B, what):
    if length % (K * B):
        raise ValueError(f"{what}: local extent {length} must be a multiple of K*B = {K}*{B}")


def meshslice_os(mesh: Mesh, X, W, K=4, B=8):
    """Y = sum over slices of  AG_col(X[:, slice]) @ AG_row(W[slice, :])."""
    _check_div(X.shape[1], K, B, "MeshSlice OS (X columns)")
    _check_div(W.shape[0], K, B, "MeshSlice OS (W rows)")
    Xs = X.map(lambda x: x.reshape(x.shape[0], -1, K, B))
    Ws = W.map(lambda w: w.reshape(-1, K, B, w.shape[1]))
    Y = None
    for kk in range(K):
        Xk = mesh.all_gather(Xs.map(lambda x: x[:, :, kk, :].reshape(x.shape[0], -1)), "col", 1)
        Wk = mesh.all_gather(Ws.map(lambda w: w[:, kk, :, :].reshape(-1, w.shape[3])), "row", 0)
        Yk = mesh.map(lambda r, c, x, w: _mm(x, w), Xk, Wk)
        Y = Yk if Y is None else Y + Yk
    return Y


def meshslice_ls(mesh: Mesh, X, W, K=4, B=8):
    """Per slice: AG_row of W rows, X @ Wk^T, reduce-scatter over the mesh row into slot kk."""
    C = mesh.C
    _check_div(W.shape[0], K, B, "MeshSlice LS (W rows)")
    O = W.shape[0] * mesh.R
    if O % (K * B * C):
        raise ValueError(f"MeshSlice LS: output width {O} must be a multiple of K*B*C")
    Ws = W.map(lambda w: w.reshape(-1, K, B, w.shape[1]))
    outs = []
    for kk in range(K):
        Wk = mesh.all_gather(Ws.map(lambda w: w[:, kk, :, :].reshape(-1, w.shape[3])), "row", 0)
        Yk = mesh.map(lambda r, c, x, w: _mm(x, w.t()), X, Wk)      # [m, O/K], partial over cols
        outs.append(mesh.reduce_scatter(Yk, "col", 1))               # [m, O/(K*C)]
    def assemble(r, c, *ys):
        m = ys[0].shape[0]
        y4 = torch.stack([y.reshape(m, -1, B) for y in ys], dim=2)   # [m, O/(K*B*C), K, B]
        return y4.reshape(m, -1)
    return mesh.map(assemble, *outs)


def meshslice_rs(mesh: Mesh, X, W, K=4, B=8):
    """Per slice: AG_col of X columns, Xk^T @ W, reduce-scatter over the mesh column."""
    R = mesh.R
    _check_div(X.shape[1], K, B, "MeshSlice RS (X columns)")
    N = X.shape[1] * mesh.C
    if N % (K * B * R):
        raise ValueError(f"MeshSlice RS: output height {N} must be a multiple of K*B*R")
    Xs = X.map(lambda x: x.reshape(x.shape[0], -1, K, B))
    outs = []
    for kk in range(K):
        Xk = mesh.all_gather(Xs.map(lambda x: x[:, :, kk, :].reshape(x.shape[0], -1)), "col", 1)
        Yk = mesh.map(lambda r, c, x, w: _mm(x.t(), w), Xk, W)      # [N/K, n], partial over rows
        outs.append(mesh.reduce_scatter(Yk, "row", 0))               # [N/(K*R), n]
    def assemble(r, c, *ys):
        n = ys[0].shape[1]
        y4 = torch.stack([y.reshape(-1, B, n) for y in ys], dim=1)   # [N/(K*B*R), K, B, n]
        return y4.reshape(-1, n)
    return mesh.map(assemble, *outs)


# ----------------------------------------------------------------------------------------------
# Wang et al. collective matmul: bidirectional ring along the mesh row
# ----------------------------------------------------------------------------------------------
def _even_halves(t, dim: int, what: str):
    """The bidirectional ring moves two halves of a shard in opposite directions."""
    for s in t.shards.values():
        if s.shape[dim] % 2:
            raise ValueError(f"wang: the {what} of a shard ({s.shape[dim]}) must be even (two half blocks)")


def wang_os(mesh: Mesh, X, W, K=1, B=8):
    n = mesh.C
    _even_halves(X, 1, "contraction length")
    Wj = mesh.all_gather(W, "row", 0)
    def blk(w, i, hi):
        h = w.shape[0] // n // 2
        return w[(2 * i + hi) * h:(2 * i + hi + 1) * h]
    lo = X.map(lambda x: x[:, :x.shape[1] // 2].contiguous())
    hi = X.map(lambda x: x[:, x.shape[1] // 2:].contiguous())
    out = mesh.map(lambda r, c, l, h, w: _mm(l, blk(w, c, 0)) + _mm(h, blk(w, c, 1)), lo, hi, Wj)
    for ii in range(1, n):
        lo = mesh.permute(lo, "col", +1)
        hi = mesh.permute(hi, "col", -1)
        out = mesh.map(lambda r, c, o, l, h, w: o + _mm(l, blk(w, (c - ii) % n, 0)) + _mm(h, blk(w, (c + ii) % n, 1)),
                       out, lo, hi, Wj)
    return out


def wang_ls(mesh: Mesh, X, W, K=1, B=8):
    n = mesh.C
    Wj = mesh.all_gather(W, "row", 0)
    def blk(w, i, hi):
        h = w.shape[0] // n // 2
        return w[(2 * i + hi) * h:(2 * i + hi + 1) * h]
    ylo = mesh.map(lambda r, c, x, w: _mm(x, blk(w, (c - 1) % n, 0).t()), X, Wj)
    yhi = mesh.map(lambda r, c, x, w: _mm(x, blk(w, (c + 1) % n, 1).t()), X, Wj)
    for ii in range(1, n):
        ylo = mesh.permute(ylo, "col", +1)
        yhi = mesh.permute(yhi, "col", -1)
        ylo = mesh.map(lambda r, c, y, x, w: y + _mm(x, blk(w, (c - ii - 1) % n, 0).t()), ylo, X, Wj)
        yhi = mesh.map(lambda r, c, y, x, w: y + _mm(x, blk(w, (c + ii + 1) % n, 1).t()), yhi, X, Wj)
    return mesh.map(lambda r, c, a, b: torch.cat([a, b], dim=1), ylo, yhi)


def wang_rs(mesh: Mesh, X, W, K=1, B=8):
    """Ring all-gather of X fused with the matmul, then reduce-scatter over the mesh column
    (the live branch of the reference, TensorParallel.py:123-149)."""
    n = mesh.C
    ml = X.shape[1]
    h = ml // 2
    def first(r, c, x, w):
        Y = torch.zeros(ml * n, w.shape[1], dtype=x.dtype, device=x.device)
        Y[2 * c * h:2 * c * h + ml] = _mm(x.t(), w)
        return Y
    Y = mesh.map(first, X, W)
    lo = mesh.permute(X.map(lambda x: x[:, :h].contiguous()), "col", +1)
    hi = mesh.permute(X.map(lambda x: x[:, h:].contiguous()), "col", -1)
    for ii in range(1, n):
        def step(r, c, y, l, hh, w, ii=ii):
            y = y.clone()
            a = 2 * ((c - ii) % n) * h
            y[a:a + h] = _mm(l.t(), w)
            b = 2 * ((c + ii) % n) * h + h
            y[b:b + h] = _mm(hh.t(), w)
            return y
        Y = mesh.map(step, Y, lo, hi, W)
        lo = mesh.permute(lo, "col", +1)
        hi = mesh.permute(hi, "col", -1)
    return mesh.reduce_scatter(Y, "row", 0)


# ----------------------------------------------------------------------------------------------
# Cannon (square meshes): skew by selection, then N-1 four-direction half-block shifts
# ----------------------------------------------------------------------------------------------
def _square(mesh):
    if mesh.R != mesh.C:
        raise ValueError("Cannon's algorithm needs a square mesh")
    return mesh.R


def cannon_os(mesh: Mesh, X, W, K=1, B=8):
    n = _square(mesh)
    Xi = mesh.all_gather(X, "col", 1)
    Wj = mesh.all_gather(W, "row", 0)
    def pick_cols(r, c, x, hi):
        h = x.shape[1] // n // 2
        k = (c + r) % n
        return x[:, (2 * k + hi) * h:(2 * k + hi + 1) * h].contiguous()
    def pick_rows(r, c, w, hi):
        h = w.shape[0] // n // 2
        k = (c + r) % n
        return w[(2 * k + hi) * h:(2 * k + hi + 1) * h].contiguous()
    xl = mesh.map(partial(pick_cols, hi=0), Xi)
    xh = mesh.map(partial(pick_cols, hi=1), Xi)
    wl = mesh.map(partial(pick_rows, hi=0), Wj)
    wh = mesh.map(partial(pick_rows, hi=1), Wj)
    out = mesh.map(lambda r, c, a, b, d, e: _mm(a, d) + _mm(b, e), xl, xh, wl, wh)
    for _ in range(1, n):
        wl, wh = mesh.permute(wl, "row", -1), mesh.permute(wh, "row", +1)
        xl, xh = mesh.permute(xl, "col", -1), mesh.permute(xh, "col", +1)
        out = mesh.map(lambda r, c, o, a, b, d, e: o + _mm(a, d) + _mm(b, e), out, xl, xh, wl, wh)
    return out


def cannon_ls(mesh: Mesh, X, W, K=1, B=8):
    n = _square(mesh)
    h = W.shape[0] // 2
    Wj = mesh.all_gather(W, "row", 0)
    def pick(r, c, w, hi):
        k = (c + r) % n
        return w[(2 * k + hi) * h:(2 * k + hi + 1) * h].contiguous()
    wl = mesh.map(partial(pick, hi=0), Wj)
    wh = mesh.map(partial(pick, hi=1), Wj)
    yl = mesh.map(lambda r, c, x, w: _mm(x, w.t()), X, wl)
    yh = mesh.map(lambda r, c, x, w: _mm(x, w.t()), X, wh)
    for _ in range(1, n):
        wl, wh = mesh.permute(wl, "row", -1), mesh.permute(wh, "row", +1)
        yl, yh = mesh.permute(yl, "col", -1), mesh.permute(yh, "col", +1)
        yl = mesh.map(lambda r, c, y, x, w: y + _mm(x, w.t()), yl, X, wl)
        yh = mesh.map(lambda r, c, y, x, w: y + _mm(x, w.t()), yh, X, wh)
    yl, yh = mesh.permute(yl, "col", -1), mesh.permute(yh, "col", +1)
    Yik = mesh.map(lambda r, c, a, b: torch.cat([a, b], dim=1), yl, yh)
    Yi = mesh.all_gather(Yik, "col", 1)
    return mesh.map(lambda r, c, y: y[:, 2 * ((c - r) % n) * h:2 * ((c - r) % n) * h + 2 * h].contiguous(), Yi)


def cannon_rs(mesh: Mesh, X, W, K=1, B=8):
    n = _square(mesh)
    h = X.shape[1] // 2
    Xi = mesh.all_gather(X, "col", 1)
    def pick(r, c, x, hi):
        k = (c + r) % n
        return x[:, (2 * k + hi) * h:(2 * k + hi + 1) * h].contiguous()
    xl = mesh.map(partial(pick, hi=0), Xi)
    xh = mesh.map(partial(pick, hi=1), Xi)
    yl = mesh.map(lambda r, c, x, w: _mm(x.t(), w), xl, W)
    yh = mesh.map(lambda r, c, x, w: _mm(x.t(), w), xh, W)
    for _ in range(1, n):
        xl, xh = mesh.permute(xl, "col", -1), mesh.permute(xh, "col", +1)
        yl, yh = mesh.permute(yl, "row", -1), mesh.permute(yh, "row", +1)
        yl = mesh.map(lambda r, c, y, x, w: y + _mm(x.t(), w), yl, xl, W)
        yh = mesh.map(lambda r, c, y, x, w: y + _mm(x.t(), w), yh, xh, W)
    yl, yh = mesh.permute(yl, "row", -1), mesh.permute(yh, "row", +1)
    Ykj = mesh.map(lambda r, c, a, b: torch.cat([a, b], dim=0), yl, yh)
    Yj = mesh.all_gather(Ykj, "row", 0)
    return mesh.map(lambda r, c, y: y[2 * ((r - c) % n) * h:2 * ((r - c) % n) * h + 2 * h].contiguous(), Yj)


# ----------------------------------------------------------------------------------------------
# SUMMA: lcm(R, C) panel steps of broadcast (+ reduce)
# ----------------------------------------------------------------------------------------------
def summa_os(mesh: Mesh, X, W, K=1, B=8):
    steps = math.lcm(mesh.R, mesh.C)
    kl, kr = X.shape[1], W.shape[0]
    Kd = kl * mesh.C
    p = Kd // steps
    Y = None
    for s in range(steps):
        k0 = s * p
        cx, rx = k0 // kl, k0 // kr
        Xp = mesh.broadcast(X.map(lambda x: x[:, k0 - cx * kl:k0 - cx * kl + p].contiguous()), "col", cx)
        Wp = mesh.broadcast(W.map(lambda w: w[k0 - rx * kr:k0 - rx * kr + p].contiguous()), "row", rx)
        Yk = mesh.map(lambda r, c, x, w: _mm(x, w), Xp, Wp)
        Y = Yk if Y is None else Y + Yk
    return Y


def summa_ls(mesh: Mesh, X, W, K=1, B=8):
    steps = math.lcm(mesh.R, mesh.C)
    nr = W.shape[0]
    N = nr * mesh.R
    nc = N // mesh.C
    p = N // steps
    pieces = []
    for s in range(steps):
        n0 = s * p
        rw, co = n0 // nr, n0 // nc
        Wp = mesh.broadcast(W.map(lambda w: w[n0 - rw * nr:n0 - rw * nr + p].contiguous()), "row", rw)
        Yp = mesh.reduce_to(mesh.map(lambda r, c, x, w: _mm(x, w.t()), X, Wp), "col", co)
        pieces.append((co, Yp))
    def assemble(r, c, *ys):
        return torch.cat([y for (co, _), y in zip(pieces, ys) if co == c], dim=1)
    return mesh.map(assemble, *[y for _, y in pieces])


def summa_rs(mesh: Mesh, X, W, K=1, B=8):
    steps = math.lcm(mesh.R, mesh.C)
    ml = X.shape[1]
    M = ml * mesh.C
    mr = M // mesh.R
    p = M // steps
    pieces = []
    for s in range(steps):
        m0 = s * p
        cx, ro = m0 // ml, m0 // mr
        Xp = mesh.broadcast(X.map(lambda x: x[:, m0 - cx * ml:m0 - cx * ml + p].contiguous()), "col", cx)
        Yp = mesh.reduce_to(mesh.map(lambda r, c, x, w: _mm(x.t(), w), Xp, W), "row", ro)
        pieces.append((ro, Yp))
    def assemble(r, c, *ys):
        return torch.cat([y for (ro, _), y in zip(pieces, ys) if ro == r], dim=0)
    return mesh.map(assemble, *[y for _, y in pieces])


ALGORITHMS = {
    "collective": (collective_os, collective_ls, collective_rs),
    "wang": (wang_os, wang_ls, wang_rs),
    "cannon": (cannon_os, cannon_ls, cannon_rs),
    "summa": (summa_os, summa_ls, summa_rs),
    "meshslice": (meshslice_os, meshslice_ls, meshslice_rs),
    "meshflow": (meshslice_os, meshslice_ls, meshslice_rs),
}


class SPMD:
    """Builder of the three dataflows of one algorithm on one mesh (TensorParallel.py:346-377).

    ``backend='auto'`` uses the fused tcgen05 kernels for 'meshslice' when the mesh is a GPU
    ``DistMesh`` with an attached fused engine, and the generic collective formulation
    otherwise; ``backend='collective'`` forces the generic formulation (the NCCL baseline).
    """

    def __init__(self, mesh: Mesh, algorithm: str = "collective", blocksize: int = 8, jit: bool = True,
                 backend: str = "auto"):
        self.mesh = mesh
        self.algorithm = algorithm if algorithm in ALGORITHMS else "meshslice"
        self.blocksize = blocksize
        self.backend = backend
        if self.algorithm == "cannon" and mesh.R != mesh.C:
            raise ValueError("Cannon's algorithm needs a square mesh")
        self.funcs = dict(zip(("os", "ls", "rs"), ALGORITHMS[self.algorithm]))

    def _fused(self):
        eng = getattr(self.mesh, "engine", None)
        if self.backend == "collective" or eng is None or self.algorithm not in ("meshslice", "meshflow"):
            return None
        return eng

    def _build(self, which: str, K: int) -> Callable:
        eng = self._fused()
        ring_eng = getattr(self.mesh, "engine", None)
        if (eng is None and self.backend != "collective" and which == "os" and hasattr(ring_eng, "os_kpanel")
                and self.algorithm in ("summa", "wang", "cannon")):
            # the OS product of the baseline algorithms on the fused kernel's K-panel schedule
            mesh, order = self.mesh, self.algorithm
            def run_panels(X, W, **kw):
                y = ring_eng.os_kpanel(X, W, order=order, sub=max(1, K), **kw)
                return ShardedTensor(mesh, {mesh.coords()[0]: y}) if isinstance(X, ShardedTensor) else y
            return run_panels
        if (eng is None and self.backend != "collective" and which in ("ls", "rs") and hasattr(ring_eng, "os_kpanel")
                and self.algorithm in ("summa", "wang", "cannon")):
            # LS / RS of the baseline algorithms as schedules of the fused kernel.  What travels in
            # their rings is the OUTPUT: Wang's two accumulators visit the ranks one after the other
            # and end at their owner, Cannon does the same from a skewed start, SUMMA reduces one
            # panel per step to its owner.  On a switch a ring hop is a direct store to the owner, so
            # each is the push epilogue with the algorithm's own order of owners and granularity:
            #   wang    one monolithic gather, owners visited from the next rank on (rotation by rank)
            #   cannon  the same from the skewed start (r + c)
            #   summa   lcm(R, C) * K panels, every rank walks the owners in the same step order
            mesh, alg = self.mesh, self.algorithm
            fn = getattr(ring_eng, which)
            if alg == "summa":
                sched = dict(n_slices=math.lcm(mesh.R, mesh.C) * max(1, K), rot_index=-1)
            elif alg == "wang":
                sched = dict(n_slices=1, rot_index=None)
            else:
                sched = dict(n_slices=1, rot_index=getattr(mesh, "r", 0) + getattr(mesh, "c", 0))
            def run_ring(X, W, **kw):
                y = fn(X, W, **sched, **kw)
                return ShardedTensor(mesh, {mesh.coords()[0]: y}) if isinstance(X, ShardedTensor) else y
            return run_ring
        if eng is not None:
            fn, mesh = getattr(eng, which), self.mesh
            def run(X, W, **kw):
                y = fn(X, W, n_slices=K, **kw)
                return ShardedTensor(mesh, {mesh.coords()[0]: y}) if isinstance(X, ShardedTensor) else y
            return run
        return partial(self.funcs[which], self.mesh, K=K, B=self.blocksize)

    def OS(self, K: int = 8):
        return self._build("os", K)

    def LS(self, K: int = 8):
        return self._build("ls", K)

    def RS(self, K: int = 8):
        return self._build("rs", K)


INIT_TILE = 256      # edge of the square tiles that random initial values are drawn in


def init_block(global_shape, std: float, seed: int, r0: int, r1: int, c0: int, c1: int, device=None) -> torch.Tensor:
    """Rows [r0, r1) x columns [c0, c1) of a virtual global N(0, std) fp32 matrix of ``global_shape``.

    The global matrix is defined tile by tile: tile (i, j) of INIT_TILE x INIT_TILE elements is
    drawn from its own generator, seeded by (seed, i, j).  A block is assembled from the tiles it
    touches, so its values do not depend on how the matrix is cut: every mesh shape initialises
    the same model, and no rank ever materialises more than its own block (plus tile borders)."""
    d0, d1 = global_shape
    on_gpu = device is not None and torch.device(device).type == "cuda"
    dev = device if on_gpu else "cpu"
    out = torch.empty(r1 - r0, c1 - c0, dtype=torch.float32, device=dev)
    T = INIT_TILE
    g = torch.Generator(device=dev)
    tiles_j = (d1 + T - 1) // T
    for i in range(r0 // T, (r1 - 1) // T + 1):
        for j in range(c0 // T, (c1 - 1) // T + 1):
            g.manual_seed((seed * 1000003 + i * tiles_j + j) * 2654435761 % (1 << 62))
            tile = torch.randn(T, T, generator=g, device=dev, dtype=torch.float32)
            a0, a1 = max(r0, i * T), min(r1, (i + 1) * T)
            b0, b1 = max(c0, j * T), min(c1, (j + 1) * T)
            out[a0 - r0:a1 - r0, b0 - c0:b1 - c0] = tile[a0 - i * T:a1 - i * T, b0 - j * T:b1 - j * T]
    if std != 1.0:
        out *= std
    return out


def createMultihostMatrix(mesh: Mesh, global_shape, dtype=torch.bfloat16, seed: int = 0, device=None,
                          std: float = 1.0) -> ShardedTensor:
    """Random N(0, std) matrix block-sharded P(row, col) (TensorParallel.py:419-423).  No rank
    materialises the global matrix, and (unlike the reference, which seeds by process index)
    the global values do not depend on the mesh shape: see ``init_block``."""
    d0, d1 = global_shape
    if d0 % mesh.R or d1 % mesh.C:
        raise ValueError(f"shape {tuple(global_shape)} not divisible by mesh {mesh.shape}")
    b0, b1 = d0 // mesh.R, d1 // mesh.C
    shards = {}
    for (r, c) in mesh.coords():
        t = init_block(global_shape, std, seed, r * b0, (r + 1) * b0, c * b1, (c + 1) * b1, device=device)
        shards[(r, c)] = t.to(dtype).to(device) if device is not None else t.to(dtype)
    return ShardedTensor(mesh, shards)
