"""AdamW with fp32 master weights over the flat parameter buffers of a rank.

bf16 parameters are what the forward pass reads; the optimizer keeps fp32 master copies and
moments, reads bf16 (sharded weights) or fp32 (row-replicated parameters) gradients, and writes
both the master and the bf16 copy in one fused kernel per buffer.  Gradient clipping uses the
global L2 norm: sharded parameters contribute once per rank, row-replicated parameters once per
mesh column.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from . import _native


class FlatGroup:
    """One contiguous parameter buffer with its gradient buffer (same element count)."""

    def __init__(self, param: torch.Tensor, grad: torch.Tensor, kind: str):
        assert param.numel() == grad.numel() and param.numel() % 4 == 0
        self.param, self.grad, self.kind = param, grad, kind
        self.master = param.float().clone()
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)


class AdamW:
    def __init__(self, groups: List[FlatGroup], lr: float = 1e-4, betas=(0.9, 0.95), eps: float = 1e-8,
                 weight_decay: float = 0.0, max_grad_norm: Optional[float] = 1.0, mesh=None):
        self.groups, self.lr, self.betas, self.eps, self.wd = groups, lr, betas, eps, weight_decay
        self.max_grad_norm, self.mesh = max_grad_norm, mesh
        self.step_count = 0
        dev = groups[0].param.device
        self._sq = torch.zeros(2, dtype=torch.float32, device=dev)
        self._scale = torch.ones(1, dtype=torch.float32, device=dev)
        self.last_grad_norm = None

    def _grad_scale(self):
        """Device scalar that rescales the gradients so that their global norm is <= max."""
        if self.max_grad_norm is None:
            return None
        self._sq.zero_()
        for g in self.groups:
            idx = 0 if g.kind == "sharded" else 1
            if g.grad.is_cuda:
                _native.load().sumsq(g.grad.data_ptr(), 1 if g.grad.dtype == torch.float32 else 0,
                                     g.grad.numel(), self._sq[idx:idx + 1].data_ptr(), _native.stream_ptr())
            else:
                self._sq[idx] += g.grad.float().pow(2).sum()
        sq = self._sq.clone()
        if self.mesh is not None and self.mesh.R * self.mesh.C > 1 and hasattr(self.mesh, "dist"):
            d = self.mesh.dist
            if self.mesh.R > 1:
                # replicated parameters are identical along a mesh column: count them once
                sq[1] = sq[1] / self.mesh.R
            d.all_reduce(sq, group=self.mesh.group)
        norm = torch.sqrt(sq.sum())
        self.last_grad_norm = norm
        torch.clamp(self.max_grad_norm / (norm + 1e-6), max=1.0, out=self._scale[0:1]) if False else \
            self._scale.copy_(torch.clamp(self.max_grad_norm / (norm + 1e-6), max=1.0).reshape(1))
        return self._scale

    def step(self):
        self.step_count += 1
        b1, b2 = self.betas
        bc1, bc2 = 1 - b1 ** self.step_count, 1 - b2 ** self.step_count
        scale = self._grad_scale()
        for g in self.groups:
            if g.param.is_cuda:
                _native.load().adamw_step(g.param.data_ptr(), g.master.data_ptr(), g.m.data_ptr(), g.v.data_ptr(),
                                          g.grad.data_ptr(), 1 if g.grad.dtype == torch.float32 else 0,
                                          g.param.numel(), self.lr, b1, b2, self.eps, self.wd, bc1, bc2,
                                          0 if scale is None else scale.data_ptr(), _native.stream_ptr())
            else:
                gr = g.grad.float() * (1.0 if scale is None else scale.item())
                g.m.mul_(b1).add_(gr, alpha=1 - b1)
                g.v.mul_(b2).addcmul_(gr, gr, value=1 - b2)
                upd = (g.m / bc1) / ((g.v / bc2).sqrt() + self.eps) + self.wd * g.master
                g.master.add_(upd, alpha=-self.lr)
                g.param.copy_(g.master.to(g.param.dtype))

    def zero_grad(self):
        for g in self.groups:
            g.grad.zero_()

    def resync_from_params(self, step: int = 0):
        """Rebuild the optimizer state from the current bf16 parameters: the fp32 master copies
        become the parameters, both moments are cleared and the step counter is set.  Needed after
        parameters were written behind the optimizer's back (a checkpoint without optimizer
        state, imported weights); otherwise the next step would overwrite them from the stale
        master copies."""
        self.step_count = int(step)
        for g in self.groups:
            g.master.copy_(g.param.float())
            g.m.zero_()
            g.v.zero_()

    def named_state(self, params):
        """Views of the flat master / m / v buffers per named parameter shard.

        ``params`` is ``model.parameters()``.  Returns {name: {coord: (master, m, v)}} where each
        view has the shape of the parameter shard; a parameter that does not live inside one of
        this optimizer's flat buffers is an error.  This is what makes the optimizer state
        save-able and re-shardable with the same rules as the parameters themselves."""
        out = {}
        spans = [(g, g.param.data_ptr(), g.param.data_ptr() + g.param.numel() * g.param.element_size())
                 for g in self.groups]
        for name, p, _, _ in params:
            per = {}
            for key, t in p.shards.items():
                for g, lo, hi in spans:
                    if lo <= t.data_ptr() < hi:
                        if not t.is_contiguous():
                            raise ValueError(f"{name}: parameter shard is not contiguous in its flat buffer")
                        off = (t.data_ptr() - lo) // g.param.element_size()
                        n = t.numel()
                        per[key] = tuple(b[off:off + n].view(t.shape) for b in (g.master, g.m, g.v))
                        break
                else:
                    raise ValueError(f"{name}: parameter shard {key} is outside the optimizer's flat buffers")
            out[name] = per
        return out

    def state_dict(self):
        return {"step": self.step_count,
                "groups": [{"master": g.master, "m": g.m, "v": g.v, "kind": g.kind} for g in self.groups]}

    def load_state_dict(self, sd):
        self.step_count = sd["step"]
        for g, s in zip(self.groups, sd["groups"]):
            g.master.copy_(s["master"])
            g.m.copy_(s["m"])
            g.v.copy_(s["v"])
            g.param.copy_(g.master.to(g.param.dtype))
