"""1-D tensor-parallel baselines: Wang collective-matmul (OS / IS / DP variants) and FSDP.

Counterpart of TensorParallel1D.py:25-127.  A 1-D mesh of n devices is a ``Mesh`` with R = 1;
operands are sharded along their last dimension, P(None, axis), except the FSDP input which is
sharded along its rows, P(axis, None).
"""
from __future__ import annotations

import torch

from .mesh import EmuMesh, Mesh, ShardedTensor
from .tensor_parallel import _mm


def createShardedMatrix(mesh: Mesh, global_shape, dtype=torch.bfloat16, shard_axis: int = 1, seed: int = 0,
                        device=None) -> ShardedTensor:
    """Random matrix sharded over the 1-D mesh along ``shard_axis`` (TensorParallel1D.py:14-20)."""
    g = torch.Generator().manual_seed(seed)
    full = torch.randn(*global_shape, generator=g).to(dtype)
    if device is not None:
        full = full.to(device)
    n = mesh.C
    return ShardedTensor(mesh, {(r, c): full.chunk(n, dim=shard_axis)[c].contiguous() for (r, c) in mesh.coords()})


def wang_1d_os(mesh: Mesh, X, W):
    """Y[:, shard] = X @ W[:, shard]; X's column halves travel the ring in both directions."""
    n = mesh.C
    def blk(w, i, hi):
        h = w.shape[0] // n // 2
        return w[(2 * i + hi) * h:(2 * i + hi + 1) * h]
    lo = X.map(lambda x: x[:, :x.shape[1] // 2].contiguous())
    hi = X.map(lambda x: x[:, x.shape[1] // 2:].contiguous())
    out = mesh.map(lambda r, c, l, h, w: _mm(l, blk(w, c, 0)) + _mm(h, blk(w, c, 1)), lo, hi, W)
    for i in range(1, n):
        lo, hi = mesh.permute(lo, "col", +1), mesh.permute(hi, "col", -1)
        out = mesh.map(lambda r, c, o, l, h, w: o + _mm(l, blk(w, (c - i) % n, 0)) + _mm(h, blk(w, (c + i) % n, 1)),
                       out, lo, hi, W)
    return out


def wang_1d_is(mesh: Mesh, X, W):
    """Y = X @ W^T with the contraction sharded: output halves travel the ring and accumulate."""
    n = mesh.C
    def blk(w, i, hi):
        h = w.shape[0] // n // 2
        return w[(2 * i + hi) * h:(2 * i + hi + 1) * h]
    lo = mesh.map(lambda r, c, x, w: _mm(x, blk(w, (c - 1) % n, 0).t()), X, W)
    hi = mesh.map(lambda r, c, x, w: _mm(x, blk(w, (c + 1) % n, 1).t()), X, W)
    for i in range(1, n):
        lo, hi = mesh.permute(lo, "col", +1), mesh.permute(hi, "col", -1)
        lo = mesh.map(lambda r, c, y, x, w: y + _mm(x, blk(w, (c - i - 1) % n, 0).t()), lo, X, W)
        hi = mesh.map(lambda r, c, y, x, w: y + _mm(x, blk(w, (c + i + 1) % n, 1).t()), hi, X, W)
    return mesh.map(lambda r, c, a, b: torch.cat([a, b], dim=1), lo, hi)


def wang_dp_os(mesh: Mesh, X, W):
    """Batch-sharded X [B/n, I] with row-sharded W [I/n, O]: W's halves travel the ring."""
    n = mesh.C
    def blk(x, i, hi):
        h = x.shape[1] // n // 2
        return x[:, (2 * i + hi) * h:(2 * i + hi + 1) * h]
    lo = W.map(lambda w: w[:w.shape[0] // 2].contiguous())
    hi = W.map(lambda w: w[w.shape[0] // 2:].contiguous())
    out = mesh.map(lambda r, c, x, l, h: _mm(blk(x, c, 0), l) + _mm(blk(x, c, 1), h), X, lo, hi)
    for i in range(1, n):
        lo, hi = mesh.permute(lo, "col", +1), mesh.permute(hi, "col", -1)
        out = mesh.map(lambda r, c, o, x, l, h: o + _mm(blk(x, (c - i) % n, 0), l) + _mm(blk(x, (c + i) % n, 1), h),
                       out, X, lo, hi)
    return out


def fsdp(mesh: Mesh, X, W):
    """Batch-sharded X times the all-gathered column-sharded W (TensorParallel1D.py:46-50)."""
    Wf = mesh.all_gather(W, "col", 1)
    return mesh.map(lambda r, c, x, w: _mm(x, w), X, Wf)


class SPMDWang:
    """1-D builder (TensorParallel1D.py:104-127): ``.OS``, ``.IS`` and ``.DP`` callables."""

    def __init__(self, mesh: Mesh, jit: bool = True):
        if mesh.R != 1:
            raise ValueError("SPMDWang expects a 1 x n mesh")
        self.mesh = mesh
        self.OS = lambda x, w: wang_1d_os(mesh, x, w)
        self.IS = lambda x, w: wang_1d_is(mesh, x, w)
        self.DP = lambda x, w: fsdp(mesh, x, w)
        self.DPOS = lambda x, w: wang_dp_os(mesh, x, w)
