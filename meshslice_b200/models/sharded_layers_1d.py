"""1-D parallel layers: Megatron-style tensor parallelism with Wang's collective matmul, and
FSDP (batch-sharded activations, weights sharded and gathered per layer).

Counterparts of the classes of BenchTransformer1D.py:21-116.  A 1-D arrangement of n devices is a
mesh with one axis of size one, so every layer here is the 2-D layer on a degenerate mesh and runs
on the same kernels (emulated CPU mesh, Gloo / NCCL, or the fused tcgen05 kernels):

  sharding 'tp'    mesh 1 x n: activations P(None, axis) (features / heads split), tokens whole
      dataflow 'os'   Y[:, shard] = X @ W[:, shard], X's halves travel the ring   (Wang_1DOS, :52-72)
      dataflow 'is'   Y = X @ W^T with the contraction split, the output halves travel the ring and
                      accumulate                                                 (Wang_1DIS, :74-96)
  sharding 'dp' / dataflow 'fsdp'   mesh n x 1: activations P(axis, None) (batch split), the weight
      [out, in] is split over its rows and all-gathered for the product         (FSDP, :46-50)

Backward passes follow the 2-D table (forward OS -> dX LS, dW RS, ...), which on a 1 x n mesh is the
reference's vjp of the 1-D products.
"""
from __future__ import annotations

import torch

from ..parallel.mesh import Mesh
from .sharded_layers import ShardedAttention, ShardedFFLayer, ShardedLayerNorm


def _check(mesh: Mesh, sharding: str):
    if sharding == "tp" and mesh.R != 1:
        raise ValueError("tensor-parallel 1-D layers expect a 1 x n mesh")
    if sharding == "dp" and mesh.C != 1:
        raise ValueError("batch-sharded 1-D layers expect an n x 1 mesh")


class ShardedFFLayer1D(ShardedFFLayer):
    """Linear layer of the 1-D baselines.  ``dataflow``: 'os' or 'is' (tensor parallel, 1 x n mesh,
    Wang's ring schedule) or 'fsdp' (n x 1 mesh, weight gathered)."""

    def __init__(self, mesh: Mesh, dataflow: str, in_dim: int, out_dim: int, ksplit: int = 1, **kw):
        if dataflow not in ("os", "is", "fsdp"):
            raise ValueError(f"unknown 1-D dataflow {dataflow!r}")
        _check(mesh, "dp" if dataflow == "fsdp" else "tp")
        self.dataflow_1d = dataflow
        if dataflow == "fsdp":
            # X [tokens / n, in] @ all-gather_rows(W [out / n, in])^T: the 'ls' dataflow with a
            # reduce-scatter group of one
            super().__init__(mesh, kw.pop("algorithm", "meshslice"), "ls", ksplit, in_dim, out_dim, **kw)
        else:
            super().__init__(mesh, kw.pop("algorithm", "wang"), "os" if dataflow == "os" else "ls", ksplit,
                             in_dim, out_dim, **kw)


class ShardedLayerNorm1D(ShardedLayerNorm):
    """LayerNorm without affine parameters: statistics summed over the devices when the features
    are split ('tp'), local when the batch is split ('dp')."""

    def __init__(self, mesh: Mesh, in_dim: int, sharding: str = "tp", **kw):
        _check(mesh, sharding)
        super().__init__(mesh, in_dim, affine=False, eps=1e-6, **kw)


class ShardedAttention1D(ShardedAttention):
    """Attention with the heads split over the devices ('tp') or the sequences ('dp')."""

    def __init__(self, mesh: Mesh, n_heads: int, seqlen: int, sharding: str = "tp", **kw):
        _check(mesh, sharding)
        super().__init__(mesh, n_heads, seqlen, **kw)
