"""2-D sharded layers: linear (three dataflows), LayerNorm over column-sharded features,
attention, GeLU, and the reference's Transformer block.

Sharding follows ShardedLayers.py: activations [tokens, features] are P(row, col) (tokens over
mesh rows, features over mesh columns); a linear weight is P(row, col) as well, stored
[out, in] for the 'ls' dataflow and [in, out] otherwise (ShardedLayers.py:33-36); QKV columns
are ordered per head [q | k | v] (ShardedLayers.py:152-153); LayerNorm parameters are P(col).

Every layer has an explicit ``forward`` / ``backward`` pair (the reference wires the same three
GeMMs through jax.custom_vjp, ShardedLayers.py:41-81):

    dataflow   forward        dX              dW
    'os'       OS(x, w)       LS(dy, w)       RS(x, dy)
    'ls'       LS(x, w)       OS(dy, w)       RS(dy, x)
    'rs'       RS(x, w)       LS(w, dy)       OS(x, dy)     (x arrives transposed [in, tokens])

Layers work on ``ShardedTensor`` and therefore run unchanged on the emulated CPU mesh, on a
Gloo/NCCL ``DistMesh`` and, through the mesh's fused engine, on the tcgen05 kernels.
"""
from __future__ import annotations

from typing import Callable, List, Optional

import torch

from ..ops import functional as F
from ..parallel.mesh import Mesh, ShardedTensor
from ..parallel.tensor_parallel import SPMD, createMultihostMatrix


def _default_alloc(shape, dtype, device):
    return torch.empty(shape, dtype=dtype, device=device)


class ShardedFFLayer:
    """Linear layer y = x @ W (no bias, as in the reference) sharded over both mesh axes."""

    def __init__(self, mesh: Mesh, algorithm: str, dataflow: str, ksplit: int, in_dim: int, out_dim: int,
                 blocksize: int = 8, dtype=torch.bfloat16, device=None, seed: int = 0, std: float = 1.0,
                 alloc: Optional[Callable] = None, grad_alloc: Optional[Callable] = None,
                 backend: str = "auto", grad_dtype=None):
        """``grad_dtype``: dtype of the weight-gradient buffer that micro-batches accumulate into;
        default fp32 for 16-bit weights (summing many micro-batches in bf16 loses the small ones)."""
        if dataflow not in ("os", "ls", "rs"):
            raise ValueError(f"unknown dataflow {dataflow!r}")
        self.mesh, self.algorithm, self.dataflow = mesh, algorithm, dataflow
        self.ksplit, self.blocksize = ksplit, blocksize
        self.in_dim, self.out_dim = in_dim, out_dim
        gshape = (out_dim, in_dim) if dataflow == "ls" else (in_dim, out_dim)
        init = createMultihostMatrix(mesh, gshape, dtype=dtype, seed=seed, device=device, std=std)
        if alloc is not None:
            placed = {}
            for k, v in init.shards.items():
                t = alloc(v.shape, dtype, v.device)
                t.copy_(v)
                placed[k] = t
            init = ShardedTensor(mesh, placed)
        self.weight = init
        galloc = grad_alloc or _default_alloc
        if grad_dtype is None:
            grad_dtype = torch.float32 if dtype in (torch.bfloat16, torch.float16) else dtype
        self.grad = ShardedTensor(mesh, {k: galloc(v.shape, grad_dtype, v.device).zero_() for k, v in init.shards.items()})
        b = SPMD(mesh, algorithm, blocksize, backend=backend)
        self._OS, self._LS, self._RS = b.OS(ksplit), b.LS(ksplit), b.RS(ksplit)
        self._fused = b._fused() is not None
        self._x = None

    # dW accumulates across micro-batches: the fused kernels add into the gradient buffer in
    # their epilogue / reduce phase, the generic formulation adds afterwards
    def _dw(self, fn, a: ShardedTensor, b: ShardedTensor):
        if self._fused:
            (key, g), = self.grad.shards.items()
            fn(a, b, out=g, accumulate=True)
            return
        dw = fn(a, b)
        for k, g in self.grad.shards.items():
            g += dw.shards[k]

    def forward_gelu(self, x: ShardedTensor):
        """y = gelu(x @ W) with the activation applied in the GEMM epilogue (fused 'os' layers
        only).  Returns (gelu output, pre-activation); the caller keeps the latter for backward."""
        if not (self._fused and self.dataflow == "os"):
            raise RuntimeError("forward_gelu needs a fused 'os' layer")
        self._x = x
        (key, xl), = x.shards.items()
        m, n = xl.shape[0], self.weight.shards[key].shape[1]
        pre = torch.empty(m, n, dtype=xl.dtype, device=xl.device)
        y = self._OS(x, self.weight, act="gelu", pre_act=pre)
        return y, ShardedTensor(self.mesh, {key: pre})

    def forward(self, x: ShardedTensor) -> ShardedTensor:
        self._x = x
        w = self.weight
        if self.dataflow == "os":
            return self._OS(x, w)
        if self.dataflow == "ls":
            return self._LS(x, w)
        return self._RS(x, w)

    def backward(self, dy: ShardedTensor, need_dx: bool = True) -> Optional[ShardedTensor]:
        x, w = self._x, self.weight
        self._x = None
        if self.dataflow == "os":
            self._dw(self._RS, x, dy)
            return self._LS(dy, w) if need_dx else None
        if self.dataflow == "ls":
            self._dw(self._RS, dy, x)
            return self._OS(dy, w) if need_dx else None
        self._dw(self._OS, x, dy)
        return self._LS(w, dy) if need_dx else None

    def zero_grad(self):
        for g in self.grad.shards.values():
            g.zero_()

    def parameters(self):
        return [("weight", self.weight, self.grad, "sharded")]


class ShardedLayerNorm:
    """LayerNorm over the global feature dimension of column-sharded activations, with an
    optional fused residual add: h = x (+ res), y = LN(h).  The reference's live kernel applies
    no affine transform (ShardedLayers.py:123-138); ``affine=True`` applies gamma / beta."""

    def __init__(self, mesh: Mesh, in_dim: int, affine: bool = False, eps: float = 1e-6,
                 dtype=torch.bfloat16, device=None, alloc: Optional[Callable] = None,
                 grad_alloc: Optional[Callable] = None):
        self.mesh, self.in_dim, self.affine, self.eps = mesh, in_dim, affine, eps
        local = in_dim // mesh.C
        a = alloc or _default_alloc
        mk = lambda fill: ShardedTensor(mesh, {k: a((local,), dtype, device).fill_(fill) for k in mesh.coords()})
        self.gamma, self.bias = mk(1.0), mk(0.0)
        ga = grad_alloc or _default_alloc
        z = lambda: ShardedTensor(mesh, {k: ga((local,), torch.float32, device).zero_() for k in mesh.coords()})
        self.dgamma, self.dbias = z(), z()
        self._saved = None

    def forward(self, x: ShardedTensor, res: Optional[ShardedTensor] = None):
        """Returns y; ``self.h`` holds x + res (the new residual stream)."""
        m = self.mesh
        g = self.gamma if self.affine else None
        b = self.bias if self.affine else None
        G = lambda k: g.shards[k] if g is not None else None
        Bt = lambda k: b.shards[k] if b is not None else None
        R = lambda k: res.shards[k] if res is not None else None
        if m.C == 1:
            outs = {k: F.ln_full(x.shards[k], R(k), G(k), Bt(k), self.eps) for k in m.coords()}
            h = ShardedTensor(m, {k: v[0] for k, v in outs.items()})
            y = ShardedTensor(m, {k: v[1] for k, v in outs.items()})
            mr = ShardedTensor(m, {k: v[2] for k, v in outs.items()})
        elif self._exchanger(x) is not None:
            # statistics travel inside the two kernels (peer stores + arrival counters): no collective
            (k, xl), = x.shards.items()
            prod, cons = self._exchange(xl.shape[0], xl.shape[1], backward=False)
            hl, _ = F.ln_stats(xl, R(k), exch=prod)
            h = ShardedTensor(m, {k: hl})
            outs = {k: F.ln_apply(hl, None, G(k), Bt(k), self.in_dim, self.eps, exch=cons)}
            y = ShardedTensor(m, {k: v[0] for k, v in outs.items()})
            mr = ShardedTensor(m, {k: v[1] for k, v in outs.items()})
        else:
            hs = {k: F.ln_stats(x.shards[k], R(k)) for k in m.coords()}
            h = ShardedTensor(m, {k: v[0] for k, v in hs.items()})
            stats = m.all_reduce(ShardedTensor(m, {k: v[1] for k, v in hs.items()}), "col")
            outs = {k: F.ln_apply(h.shards[k], stats.shards[k], G(k), Bt(k), self.in_dim, self.eps)
                    for k in m.coords()}
            y = ShardedTensor(m, {k: v[0] for k, v in outs.items()})
            mr = ShardedTensor(m, {k: v[1] for k, v in outs.items()})
        self.h = h
        self._saved = (h, mr)
        return y

    def _exchanger(self, t: ShardedTensor):
        """The mesh's in-kernel row exchange, when it has one and the shard lives on its GPU."""
        ex = getattr(getattr(self.mesh, "engine", None), "row_exchange", None)
        if ex is None or len(t.shards) != 1 or not next(iter(t.shards.values())).is_cuda:
            return None
        return ex

    def _exchange(self, rows: int, cols: int, backward: bool):
        from .. import _native
        grid = _native.load().ln_grid(1 if backward else 0, rows, cols)
        return self.mesh.engine.row_exchange.next(rows, grid)

    def backward(self, dy: ShardedTensor, dres: Optional[ShardedTensor] = None) -> ShardedTensor:
        """Gradient w.r.t. h; ``dres`` is the gradient that reaches h through the residual path."""
        m = self.mesh
        h, mr = self._saved
        self._saved = None
        G = lambda k: self.gamma.shards[k] if self.affine else None
        DG = lambda k: self.dgamma.shards[k] if self.affine else None
        DB = lambda k: self.dbias.shards[k] if self.affine else None
        DR = lambda k: dres.shards[k] if dres is not None else None
        if m.C == 1:
            return ShardedTensor(m, {k: F.ln_bwd_full(dy.shards[k], h.shards[k], G(k), mr.shards[k], DG(k),
                                                      DB(k), DR(k)) for k in m.coords()})
        if self._exchanger(dy) is not None:
            (k, dyl), = dy.shards.items()
            prod, cons = self._exchange(dyl.shape[0], dyl.shape[1], backward=True)
            F.ln_bwd_stats(dyl, h.shards[k], G(k), mr.shards[k], DG(k), DB(k), exch=prod)
            return ShardedTensor(m, {k: F.ln_bwd_apply(dyl, h.shards[k], G(k), mr.shards[k], None, self.in_dim,
                                                       DR(k), exch=cons)})
        stats = ShardedTensor(m, {k: F.ln_bwd_stats(dy.shards[k], h.shards[k], G(k), mr.shards[k], DG(k), DB(k))
                                  for k in m.coords()})
        stats = m.all_reduce(stats, "col")
        return ShardedTensor(m, {k: F.ln_bwd_apply(dy.shards[k], h.shards[k], G(k), mr.shards[k],
                                                   stats.shards[k], self.in_dim, DR(k)) for k in m.coords()})

    def zero_grad(self):
        for t in list(self.dgamma.shards.values()) + list(self.dbias.shards.values()):
            t.zero_()

    def parameters(self):
        if not self.affine:
            return []
        return [("gamma", self.gamma, self.dgamma, "row_replicated"),
                ("bias", self.bias, self.dbias, "row_replicated")]


class ShardedAttention:
    """Multi-head attention with sequences on mesh rows and heads on mesh columns: no
    communication (ShardedLayers.py:141-159).  The reference is non-causal; ``causal=True`` adds
    the decoder mask.  The score matrix is never written to HBM on the GPU path."""

    def __init__(self, mesh: Mesh, n_heads: int, seqlen: int, causal: bool = False, allow_fallback: bool = False,
                 seq_shard: bool = False):
        """``allow_fallback``: shapes the attention kernel does not cover (head_dim != 128 or
        seq % 128 != 0) run the eager formulation on the GPU instead of raising.
        ``seq_shard``: sequences split over the mesh rows (ring attention).  The reference keeps whole
        sequences per mesh row (ShardedLayers.py:152) and so does this layer; the flag exists so that callers
        can ask and get a clear answer instead of wrong numerics."""
        if seq_shard:
            raise NotImplementedError("sequences are kept whole per mesh row; shard the batch over rows instead")
        if n_heads % mesh.C:
            raise ValueError("heads must divide over the mesh columns")
        self.mesh, self.seqlen, self.causal, self.allow_fallback = mesh, seqlen, causal, allow_fallback
        self.heads_per_shard = n_heads // mesh.C
        self._saved = None

    def forward(self, x: ShardedTensor) -> ShardedTensor:
        outs = {}
        for k, t in x.shards.items():
            if t.shape[0] % self.seqlen:
                raise ValueError("local tokens must be whole sequences (batch divisible by mesh rows)")
            outs[k] = F.attention_fwd(t, t.shape[0] // self.seqlen, self.seqlen, self.heads_per_shard, self.causal,
                                      allow_fallback=self.allow_fallback)
        self._saved = (x, {k: v for k, v in outs.items()})
        return ShardedTensor(self.mesh, {k: v[0] for k, v in outs.items()})

    def backward(self, dy: ShardedTensor) -> ShardedTensor:
        x, outs = self._saved
        self._saved = None
        return ShardedTensor(self.mesh, {
            k: F.attention_bwd(dy.shards[k], t, outs[k][0], outs[k][1], t.shape[0] // self.seqlen, self.seqlen,
                               self.heads_per_shard, self.causal, allow_fallback=self.allow_fallback)
            for k, t in x.shards.items()})

    def parameters(self):
        return []


class GeLU:
    def __init__(self):
        self._x = None

    def remember(self, pre_activation: ShardedTensor):
        """Used when the forward pass was fused into the producing GEMM's epilogue."""
        self._x = pre_activation

    def forward(self, x: ShardedTensor) -> ShardedTensor:
        self._x = x
        return x.map(F.gelu)

    def backward(self, dy: ShardedTensor) -> ShardedTensor:
        x, self._x = self._x, None
        return ShardedTensor(x.mesh, {k: F.gelu_bwd(dy.shards[k], v) for k, v in x.shards.items()})


def _add(a: ShardedTensor, b: ShardedTensor) -> ShardedTensor:
    return ShardedTensor(a.mesh, {k: F.add(a.shards[k], b.shards[k]) for k in a.shards})


class TransformerBlock:
    """The reference's block (ShardedLayers.py:161-190):
    norm1 -> in_proj -> attn -> out_proj -> norm2(out + x) -> ff1 -> gelu -> ff2 -> norm3(out + res).
    ``forward`` keeps what ``backward(dy)`` needs, like the reference's stashed vjp closure."""

    def __init__(self, mesh: Mesh, S: int, H: int, D: int, dataflows: List[str], alg: str = "meshflow",
                 ksplits=(4, 4, 4, 4), dtype=torch.bfloat16, device=None, std: float = 1.0, causal: bool = False):
        kw = dict(dtype=dtype, device=device, std=std)
        self.mesh = mesh
        self.norm1 = ShardedLayerNorm(mesh, H * D, dtype=dtype, device=device)
        self.in_proj = ShardedFFLayer(mesh, alg, dataflows[0], ksplits[0], H * D, 3 * H * D, seed=1, **kw)
        self.attn = ShardedAttention(mesh, H, S, causal=causal)
        self.out_proj = ShardedFFLayer(mesh, alg, dataflows[1], ksplits[1], H * D, H * D, seed=2, **kw)
        self.norm2 = ShardedLayerNorm(mesh, H * D, dtype=dtype, device=device)
        self.ff1 = ShardedFFLayer(mesh, alg, dataflows[2], ksplits[2], H * D, 4 * H * D, seed=3, **kw)
        self.gelu = GeLU()
        self.ff2 = ShardedFFLayer(mesh, alg, dataflows[3], ksplits[3], 4 * H * D, H * D, seed=4, **kw)
        self.norm3 = ShardedLayerNorm(mesh, H * D, dtype=dtype, device=device)

    def _forward(self, x: ShardedTensor) -> ShardedTensor:
        out = self.norm1.forward(x)
        out = self.in_proj.forward(out)
        out = self.attn.forward(out)
        out = self.out_proj.forward(out)
        res = self.norm2.forward(out, x)          # LN(out + x)
        out = self.ff1.forward(res)
        out = self.gelu.forward(out)
        out = self.ff2.forward(out)
        return self.norm3.forward(out, res)       # LN(out + res)

    def forward(self, x: ShardedTensor) -> ShardedTensor:
        return self._forward(x)

    def backward(self, dy: ShardedTensor) -> ShardedTensor:
        d3 = self.norm3.backward(dy)              # grad of (ff2_out + res)
        d = self.ff2.backward(d3)
        d = self.gelu.backward(d)
        d = self.ff1.backward(d)
        dres = _add(d, d3)                        # res feeds ff1 and the norm3 residual
        d2 = self.norm2.backward(dres)            # grad of (out_proj_out + x)
        d = self.out_proj.backward(d2)
        d = self.attn.backward(d)
        d = self.in_proj.backward(d)
        d = self.norm1.backward(d)
        return _add(d, d2)

    def layers(self):
        return [self.norm1, self.in_proj, self.out_proj, self.norm2, self.ff1, self.ff2, self.norm3]
