"""GPT-3-like decoder on a 2-D device mesh: learned token + position embeddings, pre-LayerNorm
blocks (attention + GeLU MLP), final LayerNorm, vocabulary-parallel LM head with fused softmax
cross-entropy.  The reference stops at one Transformer block (ShardedLayers.py:161-190) and has
no embedding, head, loss or optimizer; they are added here on the same sharding rules:

  activations      [tokens, d]          P(row, col)   tokens over mesh rows, features over columns
  linear weights   [in, out]/[out, in]  P(row, col)   (dataflow 'ls' stores [out, in])
  LayerNorm, embeddings                 P(None, col)  replicated over mesh rows

All parameters of one rank live in two flat buffers ("sharded" and "row-replicated") so that
the optimizer is one kernel launch per buffer; gradients mirror them.
"""
from __future__ import annotations

import os

from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import torch

from ..ops import functional as F
from ..parallel.mesh import Mesh, ShardedTensor
from ..parallel.tensor_parallel import init_block
from .sharded_layers import GeLU, ShardedAttention, ShardedFFLayer, ShardedLayerNorm, _add

# GeLU inside the ff1 GEMM epilogue (MSB_FUSED_GELU=0 runs the stand-alone kernel instead)
_FUSE_GELU = os.environ.get("MSB_FUSED_GELU", "1") != "0"


@dataclass
class GPTConfig:
    n_layers: int = 32
    d_model: int = 4096
    n_heads: int = 32
    ffn: int = 16384
    vocab: int = 50257
    seq: int = 2048
    dataflows: Tuple[str, str, str, str] = ("os", "os", "os", "ls")   # in_proj, out_proj, ff1, ff2
    ksplits: Tuple[int, int, int, int] = (4, 4, 4, 4)
    head_ksplit: int = 4
    algorithm: str = "meshslice"
    causal: bool = True
    eps: float = 1e-5
    init_std: float = 0.02
    vocab_pad: int = 2048          # the vocabulary is padded to a multiple of this
    dtype: torch.dtype = torch.bfloat16

    @property
    def vocab_padded(self) -> int:
        return (self.vocab + self.vocab_pad - 1) // self.vocab_pad * self.vocab_pad

    def n_params(self) -> int:
        d = self.d_model
        per_layer = 3 * d * d + d * d + 2 * d * self.ffn + 4 * d
        return self.n_layers * per_layer + (self.vocab_padded + self.seq) * d + d * self.vocab_padded + 2 * d

    def flops_per_token(self) -> float:
        """Model FLOPs of one training step per token (forward + backward = 3x forward GEMMs,
        attention counted with its full S x S score matrix as the reference's block does)."""
        d = self.d_model
        gemm = 2 * (3 * d * d + d * d + 2 * d * self.ffn) * self.n_layers + 2 * d * self.vocab_padded
        attn = 4 * self.seq * d * self.n_layers * (0.5 if self.causal else 1.0)
        return 3.0 * (gemm + attn)


class GPTBlock:
    """Pre-LN decoder block: x + out_proj(attn(in_proj(LN1 x)));  h + ff2(gelu(ff1(LN2 h)))."""

    def __init__(self, mesh: Mesh, cfg: GPTConfig, idx: int, device, alloc_sharded, alloc_rep, grad_sharded,
                 grad_rep=None):
        d, df, ks = cfg.d_model, cfg.dataflows, cfg.ksplits
        self.mesh = mesh
        kw = dict(dtype=cfg.dtype, device=device, std=cfg.init_std, alloc=alloc_sharded,
                  grad_alloc=grad_sharded)
        s = idx * 16
        self.ln1 = ShardedLayerNorm(mesh, d, affine=True, eps=cfg.eps, dtype=cfg.dtype, device=device, alloc=alloc_rep,
                                    grad_alloc=grad_rep)
        self.in_proj = ShardedFFLayer(mesh, cfg.algorithm, df[0], ks[0], d, 3 * d, seed=s + 1, **kw)
        self.attn = ShardedAttention(mesh, cfg.n_heads, cfg.seq, causal=cfg.causal)
        self.out_proj = ShardedFFLayer(mesh, cfg.algorithm, df[1], ks[1], d, d, seed=s + 2, **kw)
        self.ln2 = ShardedLayerNorm(mesh, d, affine=True, eps=cfg.eps, dtype=cfg.dtype, device=device, alloc=alloc_rep,
                                    grad_alloc=grad_rep)
        self.ff1 = ShardedFFLayer(mesh, cfg.algorithm, df[2], ks[2], d, cfg.ffn, seed=s + 3, **kw)
        self.gelu = GeLU()
        self.ff2 = ShardedFFLayer(mesh, cfg.algorithm, df[3], ks[3], cfg.ffn, d, seed=s + 4, **kw)

    # A right-stationary ('rs') layer computes x^T w and therefore wants its input transposed,
    # [in, tokens] with the features over the mesh rows; its output and the gradient it returns are
    # in the usual / the transposed orientation respectively (ShardedLayers.py:69-81).  The block keeps
    # activations [tokens, features] and re-orients around such a layer.
    def _lin(self, layer, x: ShardedTensor) -> ShardedTensor:
        return layer.forward(self.mesh.transpose(x) if layer.dataflow == "rs" else x)

    def _lin_bwd(self, layer, dy: ShardedTensor) -> ShardedTensor:
        d = layer.backward(dy)
        return self.mesh.transpose(d) if layer.dataflow == "rs" else d

    def forward(self, x: ShardedTensor, delta: Optional[ShardedTensor]):
        """Input: residual stream x and a pending branch output ``delta`` (added inside LN1).
        Returns (h, mlp_out): the caller's next LayerNorm adds them."""
        y = self.ln1.forward(x, delta)            # residual stream becomes x + delta
        x = self.ln1.h
        a = self._lin(self.out_proj, self.attn.forward(self._lin(self.in_proj, y)))
        y = self.ln2.forward(a, x)                # h = x + a
        h = self.ln2.h
        if self.ff1._fused and self.ff1.dataflow == "os" and _FUSE_GELU:
            g, pre = self.ff1.forward_gelu(y)          # GeLU in the GEMM epilogue
            self.gelu.remember(pre)
        else:
            g = self.gelu.forward(self._lin(self.ff1, y))
        m = self._lin(self.ff2, g)
        return h, m

    def backward(self, dh: ShardedTensor, dm: ShardedTensor):
        """dh: gradient of the residual stream after this block, dm: gradient of the MLP output.
        Returns (dx, ddelta) for the block below."""
        d = self._lin_bwd(self.ff1, self.gelu.backward(self._lin_bwd(self.ff2, dm)))
        dh2 = self.ln2.backward(d, dh)            # gradient of h = x + a
        d = self._lin_bwd(self.in_proj, self.attn.backward(self._lin_bwd(self.out_proj, dh2)))
        dx = self.ln1.backward(d, dh2)            # gradient of x + delta
        return dx, dx

    def layers(self):
        return [self.ln1, self.in_proj, self.out_proj, self.ln2, self.ff1, self.ff2]


class GPTModel:
    def __init__(self, mesh: Mesh, cfg: GPTConfig, device=None, alloc_sharded=None, alloc_rep=None,
                 grad_sharded=None, grad_rep=None):
        self.mesh, self.cfg, self.device = mesh, cfg, device
        if cfg.d_model % mesh.C or cfg.vocab_padded % mesh.C or cfg.n_heads % mesh.C:
            raise ValueError("model width / heads / vocabulary must divide over the mesh columns")
        d, C = cfg.d_model, mesh.C
        a_rep = alloc_rep or (lambda shape, dtype, dev: torch.empty(shape, dtype=dtype, device=dev))
        g_rep = grad_rep or (lambda shape, dtype, dev: torch.empty(shape, dtype=dtype, device=dev))
        self.tok, self.pos = ShardedTensor(mesh, {}), ShardedTensor(mesh, {})
        self.dtok, self.dpos = ShardedTensor(mesh, {}), ShardedTensor(mesh, {})
        # parameters and their gradients are carved in the same order, so a parameter and its
        # gradient sit at the same offset of the flat parameter / gradient buffers
        for (r, c) in mesh.coords():
            t = a_rep((cfg.vocab_padded, d // C), cfg.dtype, device)
            t.copy_(init_block((cfg.vocab_padded, d), cfg.init_std, 900001, 0, cfg.vocab_padded,
                               c * (d // C), (c + 1) * (d // C), device=device).to(cfg.dtype))
            p = a_rep((cfg.seq, d // C), cfg.dtype, device)
            p.copy_(init_block((cfg.seq, d), cfg.init_std, 900002, 0, cfg.seq,
                               c * (d // C), (c + 1) * (d // C), device=device).to(cfg.dtype))
            self.tok.shards[(r, c)], self.pos.shards[(r, c)] = t, p
            self.dtok.shards[(r, c)] = g_rep((cfg.vocab_padded, d // C), torch.float32, device).zero_()
            self.dpos.shards[(r, c)] = g_rep((cfg.seq, d // C), torch.float32, device).zero_()
        self.blocks = [GPTBlock(mesh, cfg, i, device, alloc_sharded, alloc_rep, grad_sharded, grad_rep)
                       for i in range(cfg.n_layers)]
        self.ln_f = ShardedLayerNorm(mesh, d, affine=True, eps=cfg.eps, dtype=cfg.dtype, device=device, alloc=alloc_rep,
                                    grad_alloc=grad_rep)
        self.head = ShardedFFLayer(mesh, cfg.algorithm, "os", cfg.head_ksplit, d, cfg.vocab_padded,
                                   dtype=cfg.dtype, device=device, std=cfg.init_std, seed=777,
                                   alloc=alloc_sharded, grad_alloc=grad_sharded)
        self._saved = None

    # ------------------------------------------------------------------ parameters
    def parameters(self):
        """[(name, param ShardedTensor, grad ShardedTensor, kind)] with kind 'sharded' (unique per
        rank) or 'row_replicated' (same value along a mesh column; gradients are summed there)."""
        out = [("tok", self.tok, self.dtok, "row_replicated"), ("pos", self.pos, self.dpos, "row_replicated")]
        for i, b in enumerate(self.blocks):
            for j, l in enumerate(b.layers()):
                out += [(f"block{i}.{type(l).__name__}{j}.{n}", p, g, kind) for n, p, g, kind in l.parameters()]
        out += [(f"ln_f.{n}", p, g, k) for n, p, g, k in self.ln_f.parameters()]
        out += [(f"head.{n}", p, g, k) for n, p, g, k in self.head.parameters()]
        return out

    def zero_grad(self):
        for _, _, g, _ in self.parameters():
            for t in g.shards.values():
                t.zero_()

    # ------------------------------------------------------------------ training step pieces
    def forward_backward(self, tokens: ShardedTensor, targets: ShardedTensor, n_tokens_global: int):
        """One micro-batch: forward, loss, backward; gradients accumulate.  ``tokens`` / ``targets``
        hold, per coordinate, the int64 ids of the sequences of that mesh row [local_tokens].
        Returns the ShardedTensor of per-coordinate loss contributions (sum over local tokens of
        the token loss divided by n_tokens_global; summing over the mesh rows gives the mean)."""
        m, cfg = self.mesh, self.cfg
        x = ShardedTensor(m, {k: F.embedding_fwd(tokens.shards[k], self.tok.shards[k], self.pos.shards[k], cfg.seq)
                              for k in m.coords()})
        delta = None
        for b in self.blocks:
            x, delta = b.forward(x, delta)
        y = self.ln_f.forward(x, delta)
        logits = self.head.forward(y)                                    # [T/R, Vp/C]
        vc = cfg.vocab_padded // m.C
        ex = getattr(getattr(m, "engine", None), "row_exchange", None)
        k0 = l0 = None
        if len(logits.shards) == 1:
            (k0, l0), = logits.shards.items()
        if ex is not None and l0 is not None and l0.is_cuda:
            # max / sum-exp / target logit of the vocabulary slices travel inside the two kernels
            from .. import _native
            prod, cons = ex.next(l0.shape[0], _native.load().ce_grid(l0.shape[0]))
            F.ce_partial(l0, targets.shards[k0], k0[1] * vc, cfg.vocab, exch=prod)
            row_loss = F.ce_grad_exchanged_(l0, targets.shards[k0], k0[1] * vc, cfg.vocab, 1.0 / n_tokens_global, cons)
            loss = ShardedTensor(m, {k0: row_loss.sum() / n_tokens_global})
        else:
            parts = {k: F.ce_partial(logits.shards[k], targets.shards[k], k[1] * vc, cfg.vocab) for k in m.coords()}
            mx = ShardedTensor(m, {k: v[0] for k, v in parts.items()})
            gmax = m.all_reduce(mx, "col", op="max")
            se = ShardedTensor(m, {k: parts[k][1] * torch.exp(parts[k][0] - gmax.shards[k]) for k in m.coords()})
            packed = m.all_reduce(ShardedTensor(m, {k: torch.stack([se.shards[k], parts[k][2]]) for k in m.coords()}), "col")
            loss = ShardedTensor(m, {k: (torch.log(packed.shards[k][0]) + gmax.shards[k] - packed.shards[k][1]).sum()
                                     / n_tokens_global for k in m.coords()})
            # backward
            for k in m.coords():
                F.ce_grad_(logits.shards[k], targets.shards[k], k[1] * vc, cfg.vocab, gmax.shards[k],
                           packed.shards[k][0].contiguous(), 1.0 / n_tokens_global)
        d = self.head.backward(logits)
        dx = self.ln_f.backward(d)                                       # gradient of x + delta
        dh, dm = dx, dx
        for b in reversed(self.blocks):
            dh, dm = b.backward(dh, dm)
        for k in m.coords():
            F.embedding_bwd(tokens.shards[k], dh.shards[k], self.dtok.shards[k], self.dpos.shards[k], cfg.seq)
        return loss

    def sync_replicated_grads(self):
        """Sum the gradients of row-replicated parameters over the mesh rows."""
        for _, _, g, kind in self.parameters():
            if kind == "row_replicated" and self.mesh.R > 1:
                red = self.mesh.all_reduce(g, "row")
                for k in g.shards:
                    g.shards[k].copy_(red.shards[k])
