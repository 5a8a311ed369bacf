"""Stand-alone peer-to-peer collectives on the symmetric heap (the kernels of csrc/comm/p2p.cu)
with NCCL twins for comparison.  They are the B200 counterparts of the collectives that
BenchCollectives2D.py:16-26 times, along either mesh axis and on either tensor dimension.

All-gather and send-recv PUSH by default: a rank reads its own input once and writes it into the
output buffer of every peer (posted stores over NVLink, which do not wait for a round trip the way
peer loads do); the output then lives in the symmetric heap (a view of it is returned).  With
``push=False`` they pull instead (the rank reads its peers' inputs; output is a local tensor).
Reduce-scatter pulls: every rank reads its chunk of all peers' inputs and sums it.  Inputs live in
the symmetric heap (``P2PCollectives.input``).
"""
from __future__ import annotations

from typing import List

import numpy as np
import torch

from .. import _native
from . import runtime as rt
from .mesh import DistMesh


def validate_copy_jobs(jobs) -> None:
    """The copy kernel moves whole 16-byte vectors: a job whose row size, pitches or base
    addresses are not multiples of 16 would silently drop the tail of every row or fault on a
    misaligned vector access.  Raises ValueError before anything is launched."""
    for i, (src, dst, rows, row_bytes, sp, dp) in enumerate(jobs):
        if rows <= 0 or row_bytes <= 0:
            raise ValueError(f"copy job {i}: empty ({rows} rows of {row_bytes} bytes)")
        for what, v in (("row size", row_bytes), ("source pitch", sp), ("destination pitch", dp),
                        ("source address", src), ("destination address", dst)):
            if v % 16:
                raise ValueError(f"copy job {i}: {what} {v} is not a multiple of 16 bytes "
                                 f"(bf16 rows must hold a multiple of 8 elements)")
        if sp < row_bytes or dp < row_bytes:
            raise ValueError(f"copy job {i}: pitch smaller than the row ({sp}/{dp} < {row_bytes})")


def validate_reduce(srcs, src_cols: int, out_ptr: int, out_pitch: int, rows: int, cols: int) -> None:
    """Same rule for the reduce kernel (8 bf16 per vector)."""
    if rows <= 0 or cols <= 0 or cols % 8 or src_cols % 8 or out_pitch % 8:
        raise ValueError(f"reduce: {rows} x {cols} (pitches {src_cols}/{out_pitch}) must be multiples of 8 bf16")
    if not 0 < len(srcs) <= 8:
        raise ValueError(f"reduce: {len(srcs)} sources")
    for p in list(srcs) + [out_ptr]:
        if p % 16:
            raise ValueError("reduce: buffer not 16-byte aligned")


class P2PCollectives:
    def __init__(self, mesh: DistMesh, heap: rt.SymmHeap, max_bytes: int, grid: int = 148, timeout_ns: int = 10_000_000_000):
        self.mesh, self.heap, self.grid, self.timeout_ns = mesh, heap, grid, timeout_ns
        self.C = _native.load()
        self.flags = heap.alloc(rt.FLAG_WORDS * 4)
        heap.bytes_view(self.flags, rt.FLAG_WORDS * 4).zero_()
        self.inp_off = heap.alloc(max_bytes)
        self.max_bytes = max_bytes
        self.out_off = None           # output region of the push variants, allocated on first use
        self.out_bytes = 0
        self.epoch = 0
        self.done_total = 0
        torch.cuda.synchronize()
        mesh.dist.barrier()

    def input(self, shape, dtype=torch.bfloat16) -> torch.Tensor:
        """View of the symmetric input buffer; fill it before calling a collective."""
        return self.heap.tensor(self.inp_off, shape, dtype)

    def _bar(self, grid):
        self.epoch += 1
        self.done_total += grid
        n = self.heap.world
        f = lambda q, w: self.heap.ptr(q, self.flags + 4 * w)
        return dict(n_ranks=n, my_rank=self.heap.rank, entry_flags=[f(q, rt.ENTRY0) for q in range(n)],
                    exit_flags=[f(q, rt.EXIT0) for q in range(n)], epoch=self.epoch,
                    go_flag=f(self.heap.rank, rt.GO), done_counter=f(self.heap.rank, rt.DONE),
                    done_target=self.done_total, status=_native.status().dev, timeout_ns=self.timeout_ns)

    def _peers(self, axis) -> List[int]:
        m = self.mesh
        return [m.r * m.C + c for c in range(m.C)] if axis == "col" else [r * m.C + m.c for r in range(m.R)]

    def _copy(self, jobs):
        validate_copy_jobs(jobs)
        jt, _ = rt.upload_jobs(jobs, [0, len(jobs)], torch.device("cuda", torch.cuda.current_device()))
        self.C.p2p_copy(jt.data_ptr(), len(jobs), self._bar(self.grid), self.grid, _native.stream_ptr())
        return jt

    def _out_region(self, nbytes: int) -> int:
        """Offset of the symmetric output region (same on every rank: every rank allocates it at the
        same point of its call sequence with the same size)."""
        if self.out_off is None:
            n_max = max(self.mesh.R, self.mesh.C)
            self.out_bytes = n_max * self.max_bytes
            self.out_off = self.heap.alloc(self.out_bytes)
            torch.cuda.synchronize()
            self.mesh.dist.barrier()
        if nbytes > self.out_bytes:
            raise ValueError(f"gathered output of {nbytes} bytes exceeds the output region ({self.out_bytes})")
        return self.out_off

    def all_gather(self, rows: int, cols: int, axis: str, dim: int, out: torch.Tensor = None, push: bool = True):
        """Gathers every peer's [rows, cols] bf16 input along ``axis`` and concatenates on ``dim``."""
        peers = self._peers(axis)
        n = len(peers)
        shape = (rows * n, cols) if dim == 0 else (rows, cols * n)
        if push and out is None:
            rb = cols * 2
            off = self._out_region(n * rows * rb)
            me = peers.index(self.heap.rank)
            src = self.heap.ptr(self.heap.rank, self.inp_off)
            jobs = []
            for k in range(n):           # every rank starts at a different destination
                q = peers[(me + 1 + k) % n]
                base = self.heap.ptr(q, off)
                if dim == 0:
                    jobs.append((src, base + me * rows * rb, rows, rb, rb, rb))
                else:
                    jobs.append((src, base + me * rb, rows, rb, rb, n * rb))
            self._keep = self._copy(jobs)     # the kernel's exit barrier: every rank's block has landed
            return self.heap.tensor(off, shape)
        if out is None:
            out = torch.empty(shape, dtype=torch.bfloat16, device="cuda")
        rb = cols * 2
        jobs = []
        me = peers.index(self.heap.rank)
        # every rank starts with a different peer so that no port serves all readers at once
        for k in range(n):
            i = (me + 1 + k) % n
            q = peers[i]
            src = self.heap.ptr(q, self.inp_off)
            if dim == 0:
                jobs.append((src, out.data_ptr() + i * rows * rb, rows, rb, rb, rb))
            else:
                jobs.append((src, out.data_ptr() + i * rb, rows, rb, rb, n * rb))
        self._keep = self._copy(jobs)
        return out

    def send_recv(self, rows: int, cols: int, axis: str, out: torch.Tensor = None, push: bool = True):
        """Ring shift by +1: every rank receives the input of its predecessor along ``axis``."""
        peers = self._peers(axis)
        i = peers.index(self.heap.rank)
        if push and out is None:
            rb = cols * 2
            off = self._out_region(rows * rb)
            dst = self.heap.ptr(peers[(i + 1) % len(peers)], off)
            self._keep = self._copy([(self.heap.ptr(self.heap.rank, self.inp_off), dst, rows, rb, rb, rb)])
            return self.heap.tensor(off, (rows, cols))
        src = self.heap.ptr(peers[(i - 1) % len(peers)], self.inp_off)
        if out is None:
            out = torch.empty(rows, cols, dtype=torch.bfloat16, device="cuda")
        rb = cols * 2
        self._keep = self._copy([(src, out.data_ptr(), rows, rb, rb, rb)])
        return out

    def reduce_scatter(self, rows: int, cols: int, axis: str, dim: int, out: torch.Tensor = None):
        """Sum of the peers' [rows, cols] inputs, this rank keeping its chunk along ``dim``."""
        peers = self._peers(axis)
        n = len(peers)
        i = peers.index(self.heap.rank)
        if dim == 0:
            r_, c_ = rows // n, cols
            off = i * r_ * cols * 2
        else:
            r_, c_ = rows, cols // n
            off = i * c_ * 2
        if out is None:
            out = torch.empty(r_, c_, dtype=torch.bfloat16, device="cuda")
        if rows % (n if dim == 0 else 1) or cols % (1 if dim == 0 else n):
            raise ValueError(f"reduce_scatter: {rows} x {cols} does not split {n} ways on dim {dim}")
        srcs = [self.heap.ptr(q, self.inp_off) + off for q in peers]
        validate_reduce(srcs, cols, out.data_ptr(), c_, r_, c_)
        self.C.p2p_reduce(srcs, cols, out.data_ptr(), c_, r_, c_, self._bar(self.grid), self.grid,
                          _native.stream_ptr())
        return out

    def barrier(self):
        self.C.p2p_barrier(self._bar(1), _native.stream_ptr())
