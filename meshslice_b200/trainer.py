"""Training driver: builds the mesh, the fused engine, the GPT model on flat parameter buffers
and the optimizer, and runs optimizer steps over micro-batches.

One process per GPU (``torchrun``); rank = r * C + c on an R x C mesh.  The global batch is split
over the mesh rows (whole sequences per row); every rank of a mesh row receives the same token
ids.  A step is: for each micro-batch forward + loss + backward (gradients accumulate), sum the
gradients of row-replicated parameters over the mesh rows, clip, AdamW.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from . import _native
from .models.gpt import GPTConfig, GPTModel
from .optim import AdamW, FlatGroup
from .parallel.mesh import DistMesh, EmuMesh, Mesh, ShardedTensor


class Arena:
    """Carves tensors out of one flat buffer, 128-element aligned, in call order."""

    def __init__(self, buf: torch.Tensor):
        self.buf, self.top = buf, 0

    def alloc(self, shape, dtype, device=None):
        n = int(torch.Size(shape).numel())
        assert dtype == self.buf.dtype, (dtype, self.buf.dtype)
        off = self.top
        self.top = off + (n + 127) // 128 * 128
        if self.top > self.buf.numel():
            raise MemoryError("parameter arena too small")
        return self.buf[off:off + n].view(*shape)


def param_elems(cfg: GPTConfig, R: int, C: int) -> Tuple[int, int]:
    """Elements (with alignment padding) of the sharded and row-replicated buffers of one rank."""
    pad = lambda n: (n + 127) // 128 * 128
    d, f, V = cfg.d_model, cfg.ffn, cfg.vocab_padded
    per_layer = pad(d * 3 * d // (R * C)) + pad(d * d // (R * C)) + 2 * pad(d * f // (R * C))
    sharded = cfg.n_layers * per_layer + pad(d * V // (R * C))
    rep = pad(V * d // C) + pad(cfg.seq * d // C) + (2 * cfg.n_layers + 1) * 2 * pad(d // C)
    return sharded, rep


def choose_mesh(world: int) -> Tuple[int, int]:
    """Default mesh shape per GPU count: 1x1, 1x2, 2x2, 2x4 (2 rows x 4 columns at 8 GPUs)."""
    return {1: (1, 1), 2: (1, 2), 4: (2, 2), 8: (2, 4)}.get(world, (1, world))


@dataclass
class TrainConfig:
    global_batch: int = 32
    micro_batch: int = 4          # sequences per mesh row per micro-batch
    lr: float = 1e-4
    betas: Tuple[float, float] = (0.9, 0.95)
    weight_decay: float = 0.0
    max_grad_norm: Optional[float] = 1.0
    backend: str = "fused"        # 'fused' (tcgen05 + in-kernel NVLink) or 'collective' (NCCL + library GEMM)
    timeout_ns: int = 20_000_000_000


def workspace_bytes(cfg, micro_batch: int, R: int, C: int):
    """Staging (gathered A / B operands) and slot (pushed partial tiles) bytes that the fused
    kernels of one micro-batch need, over the forward, dX and dW products of every linear layer
    under its dataflow (m = tokens per mesh row and micro-batch).  Returns (stage_a, stage_b, slots)."""
    m = micro_batch * cfg.seq
    d, f, V = cfg.d_model, cfg.ffn, cfg.vocab_padded
    lin = [(d, 3 * d, cfg.dataflows[0]), (d, d, cfg.dataflows[1]), (d, f, cfg.dataflows[2]),
           (f, d, cfg.dataflows[3]), (d, V, "os")]
    sa = sb = sl = 0
    for i, o, df in lin:
        if df == "os":      # OS(x, w), LS(dy, w), RS(x, dy)
            a, b, s_ = m * i, i * o // C, max(m * i, i * o // C)
        elif df == "ls":    # LS(x, w), OS(dy, w), RS(dy, x)
            a, b, s_ = m * o, o * i // C, max(m * o, o * i // C)
        else:               # RS(x^T, w), LS(w, dy), OS(x^T, dy): the token dimension is gathered whole
            a, b, s_ = m * i, max(i * o // C, m * R * o // C), max(m * i, m * R * o // C)
        sa, sb, sl = max(sa, a), max(sb, b), max(sl, s_)
    return 2 * sa, 2 * sb, 2 * sl


class Trainer:
    def __init__(self, cfg: GPTConfig, tcfg: TrainConfig, mesh_shape: Optional[Tuple[int, int]] = None,
                 device: Optional[torch.device] = None):
        import torch.distributed as dist
        self.cfg, self.tcfg = cfg, tcfg
        self.distributed = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size() if self.distributed else 1
        self.rank = dist.get_rank() if self.distributed else 0
        R, C = mesh_shape or choose_mesh(self.world)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        if self.distributed and self.world > 1:
            self.mesh = DistMesh(R, C)
        else:
            self.mesh = EmuMesh(1, 1)
        self.R, self.C = R, C
        self.r, self.c = (self.mesh.r, self.mesh.c) if isinstance(self.mesh, DistMesh) else (0, 0)
        if tcfg.global_batch % R or (tcfg.global_batch // R) % tcfg.micro_batch:
            raise ValueError("global batch must split into whole micro-batches per mesh row")
        self.rows_batch = tcfg.global_batch // R
        self.n_micro = self.rows_batch // tcfg.micro_batch
        n_sh, n_rep = param_elems(cfg, R, C)
        self.engine = None
        sharded_buf = None
        if tcfg.backend == "fused" and self.device.type == "cuda":
            from .parallel.engine import FusedEngine, LocalGemmEngine
            if self.world > 1:
                sa, sb, sl = self._workspace_bytes()
                self.engine = FusedEngine(self.mesh, sa, sb, sl, extra_heap_bytes=n_sh * 2 + (1 << 20),
                                          timeout_ns=tcfg.timeout_ns, exchange_rows=tcfg.micro_batch * cfg.seq)
                sharded_buf = self.engine.heap.empty((n_sh,), torch.bfloat16)
            else:
                self.engine = LocalGemmEngine(self.mesh)
        dt = cfg.dtype
        if sharded_buf is None:
            sharded_buf = torch.empty(n_sh, dtype=dt, device=self.device)
        self.p_sh = sharded_buf.zero_()
        # gradients of 16-bit weights accumulate over the micro-batches in fp32
        gdt = torch.float32 if dt in (torch.bfloat16, torch.float16) else dt
        self.g_sh = torch.zeros(n_sh, dtype=gdt, device=self.device)
        self.p_rep = torch.zeros(n_rep, dtype=dt, device=self.device)
        self.g_rep = torch.zeros(n_rep, dtype=torch.float32, device=self.device)
        a_sh, a_gsh, a_rep, a_grep = Arena(self.p_sh), Arena(self.g_sh), Arena(self.p_rep), Arena(self.g_rep)
        self.model = GPTModel(self.mesh, cfg, device=self.device, alloc_sharded=a_sh.alloc, alloc_rep=a_rep.alloc,
                              grad_sharded=a_gsh.alloc, grad_rep=a_grep.alloc)
        self.opt = AdamW([FlatGroup(self.p_sh, self.g_sh, "sharded"), FlatGroup(self.p_rep, self.g_rep, "row_replicated")],
                         lr=tcfg.lr, betas=tcfg.betas, weight_decay=tcfg.weight_decay,
                         max_grad_norm=tcfg.max_grad_norm, mesh=self.mesh if self.world > 1 else None)
        self.n_tokens = tcfg.global_batch * cfg.seq
        self._ids_dev = torch.empty(self.rows_batch, cfg.seq + 1, dtype=torch.int64, device=self.device)
        self._loss_dev = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.step_count = 0

    # ------------------------------------------------------------------ sizing
    def _workspace_bytes(self):
        return workspace_bytes(self.cfg, self.tcfg.micro_batch, self.R, self.C)

    # ------------------------------------------------------------------ data
    def rows_of_global_batch(self, ids_global: torch.Tensor) -> torch.Tensor:
        """The sequences of this rank's mesh row out of a [global_batch, seq + 1] id tensor."""
        return ids_global[self.r * self.rows_batch:(self.r + 1) * self.rows_batch]

    # ------------------------------------------------------------------ step
    def train_step(self, ids_row: torch.Tensor, read_loss: bool = True):
        """One optimizer step.  ``ids_row``: [global_batch / R, seq + 1] int64 token ids of this
        rank's mesh row, in pinned host memory or on the device.  Returns the mean token loss as a
        float when ``read_loss`` (a device-to-host read), else the device scalar."""
        cfg, mb = self.cfg, self.tcfg.micro_batch
        if ids_row.device != self.device:
            self._ids_dev.copy_(ids_row, non_blocking=True)
            ids = self._ids_dev
        else:
            ids = ids_row
        self._loss_dev.zero_()
        key = (self.r, self.c) if isinstance(self.mesh, DistMesh) else (0, 0)
        for i in range(self.n_micro):
            chunk = ids[i * mb:(i + 1) * mb]
            tok = ShardedTensor(self.mesh, {key: chunk[:, :-1].reshape(-1)})
            tgt = ShardedTensor(self.mesh, {key: chunk[:, 1:].reshape(-1)})
            loss = self.model.forward_backward(tok, tgt, self.n_tokens)
            self._loss_dev += loss.shards[key]
        self.model.sync_replicated_grads()
        self.opt.step()
        self.opt.zero_grad()
        self.step_count += 1
        if self.world > 1 and self.R > 1:
            self.mesh.dist.all_reduce(self._loss_dev, group=self.mesh.row_groups[self.c])
        if read_loss:
            return float(self._loss_dev.item())
        return self._loss_dev

    def check(self, all_ranks: bool = False):
        """Raise if a kernel of this rank reported an error status since the last check.  With
        ``all_ranks`` the ranks first exchange their status codes (one small all-reduce), so an
        error on any rank raises on every rank, naming the rank that failed."""
        if not all_ranks or self.world == 1:
            _native.check_status()
            return
        from .utils.health import agree_on_status
        torch.cuda.synchronize()
        st = _native.status()
        code = st.read()[0]
        try:
            agree_on_status(code, device=self.device)
        finally:
            if code:
                st.clear()

    def tflops(self, ms_per_step: float) -> float:
        """Model TFLOP/s of the whole job for a measured step time."""
        return self.cfg.flops_per_token() * self.n_tokens / (ms_per_step * 1e-3) / 1e12
