"""Local (per-shard) ops of the GPT block with two implementations each: the native sm_100a
kernel for CUDA tensors and a plain PyTorch fp32 formulation for CPU tensors (the oracle used
by the emulated-mesh tests).  Cross-device reductions are done by the callers.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from .. import _native

GELU_K0 = 0.7978845608028654
GELU_K1 = 0.044715


def _C():
    return _native.load()


def _st():
    return _native.stream_ptr()


def _p(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


# ----------------------------------------------------------------------------------------------
# LayerNorm over a possibly column-sharded feature dimension
# ----------------------------------------------------------------------------------------------
def ln_stats(x, res, exch=None) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """h = x (+ res); stats[row] = (sum h, sum h^2) over the local columns.  With ``exch`` (the
    producer descriptor of a ``RowExchanger``) the kernel publishes the statistics to the GPUs of
    the mesh row instead of returning them."""
    rows, cols = x.shape
    if x.is_cuda:
        h = torch.empty_like(x) if res is not None else x
        stats = None if exch is not None else torch.empty(rows, 2, device=x.device, dtype=torch.float32)
        _C().ln_fwd(1, x.data_ptr(), _p(res), h.data_ptr() if res is not None else 0, 0, 0, 0,
                    _p(stats), 0, rows, cols, cols, 0.0, _st(), exch)
        return h, stats
    h = x if res is None else (x.float() + res.float()).to(x.dtype)
    hf = h.float()
    return h, torch.stack([hf.sum(1), (hf * hf).sum(1)], 1)


def ln_apply(h, stats, gamma, beta, total_cols: int, eps: float, exch=None):
    """y = (h - mean) * rstd * gamma + beta from (all-reduced) statistics, or, with ``exch`` (the
    consumer descriptor), from the statistics the GPUs of the mesh row published."""
    rows, cols = h.shape
    if h.is_cuda:
        y = torch.empty_like(h)
        mr = torch.empty(rows, 2, device=h.device, dtype=torch.float32)
        _C().ln_fwd(2, h.data_ptr(), 0, 0, y.data_ptr(), _p(gamma), _p(beta), _p(stats),
                    mr.data_ptr(), rows, cols, total_cols, eps, _st(), exch)
        return y, mr
    mean = stats[:, 0] / total_cols
    var = (stats[:, 1] / total_cols - mean * mean).clamp_min(0)
    rstd = torch.rsqrt(var + eps)
    y = (h.float() - mean[:, None]) * rstd[:, None]
    if gamma is not None:
        y = y * gamma.float()
    if beta is not None:
        y = y + beta.float()
    return y.to(h.dtype), torch.stack([mean, rstd], 1)


def ln_full(x, res, gamma, beta, eps: float):
    """Single-device LayerNorm: returns (h, y, mean_rstd)."""
    rows, cols = x.shape
    if x.is_cuda:
        h = torch.empty_like(x) if res is not None else x
        y = torch.empty_like(x)
        mr = torch.empty(rows, 2, device=x.device, dtype=torch.float32)
        _C().ln_fwd(0, x.data_ptr(), _p(res), h.data_ptr() if res is not None else 0, y.data_ptr(),
                    _p(gamma), _p(beta), 0, mr.data_ptr(), rows, cols, cols, eps, _st())
        return h, y, mr
    h, stats = ln_stats(x, res)
    y, mr = ln_apply(h, stats, gamma, beta, cols, eps)
    return h, y, mr


def ln_bwd_stats(dy, h, gamma, mean_rstd, dgamma, dbeta, exch=None):
    """stats[row] = (sum g, sum g * xhat), g = dy * gamma; accumulates dgamma / dbeta (fp32).
    With ``exch`` the sums are published to the mesh row (nothing is returned)."""
    rows, cols = dy.shape
    if dy.is_cuda:
        stats = None if exch is not None else torch.empty(rows, 2, device=dy.device, dtype=torch.float32)
        _C().ln_bwd(1, dy.data_ptr(), h.data_ptr(), _p(gamma), mean_rstd.data_ptr(), 0, 0,
                    _p(stats), _p(dgamma), _p(dbeta), rows, cols, cols, _st(), exch)
        return stats
    xh = (h.float() - mean_rstd[:, :1]) * mean_rstd[:, 1:]
    d = dy.float()
    g = d * gamma.float() if gamma is not None else d
    if dgamma is not None:
        dgamma += (d * xh).sum(0)
    if dbeta is not None:
        dbeta += d.sum(0)
    return torch.stack([g.sum(1), (g * xh).sum(1)], 1)


def ln_bwd_apply(dy, h, gamma, mean_rstd, stats, total_cols: int, dres=None, exch=None):
    """dx = rstd * (g - mean(g) - xhat * mean(g * xhat)) (+ dres)."""
    rows, cols = dy.shape
    if dy.is_cuda:
        dx = torch.empty_like(dy)
        _C().ln_bwd(2, dy.data_ptr(), h.data_ptr(), _p(gamma), mean_rstd.data_ptr(), _p(dres),
                    dx.data_ptr(), _p(stats), 0, 0, rows, cols, total_cols, _st(), exch)
        return dx
    rstd = mean_rstd[:, 1:]
    xh = (h.float() - mean_rstd[:, :1]) * rstd
    g = dy.float() * gamma.float() if gamma is not None else dy.float()
    dx = rstd * (g - stats[:, :1] / total_cols - xh * stats[:, 1:] / total_cols)
    if dres is not None:
        dx = dx + dres.float()
    return dx.to(dy.dtype)


def ln_bwd_full(dy, h, gamma, mean_rstd, dgamma, dbeta, dres=None):
    rows, cols = dy.shape
    if dy.is_cuda:
        dx = torch.empty_like(dy)
        _C().ln_bwd(0, dy.data_ptr(), h.data_ptr(), _p(gamma), mean_rstd.data_ptr(), _p(dres),
                    dx.data_ptr(), 0, _p(dgamma), _p(dbeta), rows, cols, cols, _st())
        return dx
    stats = ln_bwd_stats(dy, h, gamma, mean_rstd, dgamma, dbeta)
    return ln_bwd_apply(dy, h, gamma, mean_rstd, stats, cols, dres)


# ----------------------------------------------------------------------------------------------
# GeLU (tanh approximation) and add
# ----------------------------------------------------------------------------------------------
def gelu(x):
    if x.is_cuda:
        y = torch.empty_like(x)
        _C().gelu_fwd(x.data_ptr(), y.data_ptr(), x.numel(), _st())
        return y
    return torch.nn.functional.gelu(x.float(), approximate="tanh").to(x.dtype)


def gelu_bwd(dy, x):
    if x.is_cuda:
        dx = torch.empty_like(x)
        _C().gelu_bwd(dy.data_ptr(), x.data_ptr(), dx.data_ptr(), x.numel(), _st())
        return dx
    xf = x.float()
    u = GELU_K0 * (xf + GELU_K1 * xf ** 3)
    t = torch.tanh(u)
    du = GELU_K0 * (1 + 3 * GELU_K1 * xf * xf)
    return (dy.float() * (0.5 * (1 + t) + 0.5 * xf * (1 - t * t) * du)).to(x.dtype)


def add(a, b):
    if a.is_cuda and a.dtype == torch.bfloat16 and a.numel() % 8 == 0:
        o = torch.empty_like(a)
        _C().add_bf16(a.data_ptr(), b.data_ptr(), o.data_ptr(), a.numel(), _st())
        return o
    return (a.float() + b.float()).to(a.dtype)


# ----------------------------------------------------------------------------------------------
# attention on the per-head [q | k | v] interleaved layout of the reference
# (ShardedLayers.py:152-153): qkv [batch * seq, heads * 3 * D]
# ----------------------------------------------------------------------------------------------
def _split_qkv(qkv, batch, seq, heads):
    D = qkv.shape[1] // (3 * heads)
    t = qkv.view(batch, seq, heads, 3, D)
    return t[:, :, :, 0], t[:, :, :, 1], t[:, :, :, 2], D  # each [b, s, h, D]


FALLBACKS = {"attention": 0}      # eager-PyTorch runs of an op on CUDA tensors (only with allow_fallback)


def _check_attention_shape(qkv, D: int, seq: int, allow_fallback: bool):
    """The tcgen05 attention kernels need head_dim 128 and seq % 128 == 0.  Any other shape on a GPU
    would mean a materialised S x S score matrix in eager PyTorch: refuse unless asked for."""
    if qkv.is_cuda and not (D == 128 and seq % 128 == 0):
        if not allow_fallback:
            raise ValueError(f"attention kernel needs head_dim 128 and seq % 128 == 0 (got head_dim {D}, seq {seq}); "
                             f"pass allow_fallback=True to run the eager PyTorch formulation instead")
        FALLBACKS["attention"] += 1


def attention_fwd(qkv, batch: int, seq: int, heads: int, causal: bool = False, allow_fallback: bool = False):
    """softmax(Q K^T / sqrt(D)) V per (sequence, head).  Returns (out [b*s, heads*D], lse)."""
    q, k, v, D = _split_qkv(qkv, batch, seq, heads)
    _check_attention_shape(qkv, D, seq, allow_fallback)
    if qkv.is_cuda and D == 128 and seq % 128 == 0:
        out = torch.empty(batch * seq, heads * D, dtype=qkv.dtype, device=qkv.device)
        lse = torch.empty(batch, heads, seq, dtype=torch.float32, device=qkv.device)
        _C().attention_fwd(qkv.data_ptr(), out.data_ptr(), lse.data_ptr(), batch, seq, heads,
                           1 if causal else 0, 1.0 / math.sqrt(D), _native.status().dev, _st())
        return out, lse
    qf, kf, vf = (t.permute(0, 2, 1, 3).float() for t in (q, k, v))  # [b, h, s, D]
    s = qf @ kf.transpose(-1, -2) / math.sqrt(D)
    if causal:
        s = s.masked_fill(torch.ones(seq, seq, dtype=torch.bool, device=s.device).triu(1), float("-inf"))
    lse = torch.logsumexp(s, -1)
    o = torch.softmax(s, -1) @ vf
    return o.permute(0, 2, 1, 3).reshape(batch * seq, heads * D).to(qkv.dtype), lse


def attention_bwd(dout, qkv, out, lse, batch: int, seq: int, heads: int, causal: bool = False,
                  allow_fallback: bool = False):
    """Gradient w.r.t. qkv in the same interleaved layout."""
    q, k, v, D = _split_qkv(qkv, batch, seq, heads)
    _check_attention_shape(qkv, D, seq, allow_fallback)
    if qkv.is_cuda and D == 128 and seq % 128 == 0:
        dqkv = torch.empty_like(qkv)
        delta = torch.empty(batch, heads, seq, dtype=torch.float32, device=qkv.device)
        dq_acc = torch.empty(batch, heads, seq, dtype=torch.float32, device=qkv.device)   # scratch: lse * log2(e)
        dout = dout.contiguous()
        _C().attention_bwd(qkv.data_ptr(), out.data_ptr(), dout.data_ptr(), lse.data_ptr(),
                           dqkv.data_ptr(), dq_acc.data_ptr(), delta.data_ptr(), batch, seq, heads,
                           1 if causal else 0,
                           1.0 / math.sqrt(D), _native.status().dev, _st())
        return dqkv
    qf, kf, vf = (t.permute(0, 2, 1, 3).float() for t in (q, k, v))
    do = dout.view(batch, seq, heads, D).permute(0, 2, 1, 3).float()
    of = out.view(batch, seq, heads, D).permute(0, 2, 1, 3).float()
    scale = 1.0 / math.sqrt(D)
    s = qf @ kf.transpose(-1, -2) * scale
    if causal:
        s = s.masked_fill(torch.ones(seq, seq, dtype=torch.bool, device=s.device).triu(1), float("-inf"))
    p = torch.exp(s - lse[..., None])
    dv = p.transpose(-1, -2) @ do
    dp = do @ vf.transpose(-1, -2)
    delta = (do * of).sum(-1, keepdim=True)
    ds = p * (dp - delta) * scale
    dq = ds @ kf
    dk = ds.transpose(-1, -2) @ qf
    dqkv = torch.stack([t.permute(0, 2, 1, 3) for t in (dq, dk, dv)], dim=3)  # [b, s, h, 3, D]
    return dqkv.reshape(batch * seq, heads * 3 * D).to(qkv.dtype)


# ----------------------------------------------------------------------------------------------
# vocabulary-parallel cross-entropy
# ----------------------------------------------------------------------------------------------
def ce_partial(logits, targets, col_offset: int, vocab: int, exch=None):
    """Per row: (max, sum exp(x - max), target logit or 0) over this shard's valid columns.  With
    ``exch`` the three values are published to the GPUs of the mesh row and None is returned."""
    rows, cols = logits.shape
    if logits.is_cuda:
        if exch is not None:
            _C().ce_partial(logits.data_ptr(), logits.stride(0), targets.data_ptr(), rows, cols, col_offset,
                            vocab, 0, 0, 0, _st(), exch)
            return None
        mx, se, tl = (torch.empty(rows, device=logits.device, dtype=torch.float32) for _ in range(3))
        _C().ce_partial(logits.data_ptr(), logits.stride(0), targets.data_ptr(), rows, cols, col_offset,
                        vocab, mx.data_ptr(), se.data_ptr(), tl.data_ptr(), _st())
        return mx, se, tl
    valid = max(0, min(cols, vocab - col_offset))
    lf = logits.float()[:, :valid]
    if valid == 0:
        z = torch.zeros(rows)
        return torch.full((rows,), float("-inf")), z, z.clone()
    mx = lf.max(1).values
    se = torch.exp(lf - mx[:, None]).sum(1)
    t = targets - col_offset
    inside = (t >= 0) & (t < valid)
    tl = torch.where(inside, lf.gather(1, t.clamp(0, valid - 1)[:, None])[:, 0], torch.zeros(rows))
    return mx, se, tl


def ce_grad_exchanged_(logits, targets, col_offset: int, vocab: int, scale: float, exch):
    """In place: logits <- (softmax - onehot) * scale with the global max / sum-exp combined inside
    the kernel from what the mesh row's GPUs published (``exch``: consumer descriptor).  Returns the
    per-row loss log(sum exp) - target logit [rows] (identical on every GPU of the mesh row)."""
    rows, cols = logits.shape
    row_loss = torch.empty(rows, device=logits.device, dtype=torch.float32)
    _C().ce_grad(logits.data_ptr(), logits.stride(0), targets.data_ptr(), rows, cols, col_offset, vocab,
                 0, 0, scale, _st(), row_loss.data_ptr(), exch)
    return row_loss


def ce_grad_(logits, targets, col_offset: int, vocab: int, gmax, gsum, scale: float):
    """In place: logits <- (softmax - onehot) * scale (padding columns get 0)."""
    rows, cols = logits.shape
    if logits.is_cuda:
        _C().ce_grad(logits.data_ptr(), logits.stride(0), targets.data_ptr(), rows, cols, col_offset,
                     vocab, gmax.data_ptr(), gsum.data_ptr(), scale, _st())
        return logits
    col = torch.arange(cols) + col_offset
    p = torch.exp(logits.float() - gmax[:, None]) / gsum[:, None] * scale
    p = torch.where(col[None, :] < vocab, p, torch.zeros_like(p))
    t = targets - col_offset
    inside = (t >= 0) & (t < cols)
    rows_i = torch.arange(rows)[inside]
    p[rows_i, t[inside]] -= scale
    logits.copy_(p.to(logits.dtype))
    return logits


# ----------------------------------------------------------------------------------------------
# embedding
# ----------------------------------------------------------------------------------------------
def embedding_fwd(tokens, tok_table, pos_table, seq: int):
    n = tokens.numel()
    cols = tok_table.shape[1]
    if tok_table.is_cuda:
        out = torch.empty(n, cols, dtype=tok_table.dtype, device=tok_table.device)
        _C().embedding_fwd(tokens.data_ptr(), tok_table.data_ptr(), pos_table.data_ptr(), out.data_ptr(),
                           n, seq, cols, _st())
        return out
    pos = torch.arange(n) % seq
    return (tok_table.float()[tokens.view(-1)] + pos_table.float()[pos]).to(tok_table.dtype)


def embedding_bwd(tokens, dout, dtok, dpos, seq: int):
    """dtok / dpos: fp32 accumulators."""
    n = tokens.numel()
    cols = dout.shape[1]
    if dout.is_cuda:
        _C().embedding_bwd(tokens.data_ptr(), dout.data_ptr(), dtok.data_ptr(), dpos.data_ptr(), n, seq,
                           cols, _st())
        return
    dtok.index_add_(0, tokens.view(-1), dout.float())
    dpos += dout.float().view(n // seq, seq, cols).sum(0)
