"""Runtime for the fused kernels: an IPC-shared ("symmetric") device heap, the per-rank
workspace (staging buffers, reduce slots, flags) and the addressing of peers' copies of it.

One process drives one GPU.  Every rank allocates one heap with ``cudaMalloc``, exports it as a
CUDA IPC handle, and maps every peer's heap; because all ranks carve their heaps with the same
sequence of bump allocations, "peer base + my offset" addresses the peer's copy of a buffer.
Replaces what ``jax.distributed.initialize`` + XLA's collective runtime provide to the
reference (TensorParallel.py:364-377, ShardedLayers.py:198).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np
import torch

from .. import _native

# uint32 indices inside the flag block of a workspace
ENTRY0, EXIT0, GO, DONE = 0, 8, 16, 17
RESET0 = 17            # first word cleared before every fused launch
CHUNK0, NCHUNK = 32, 160
COUNTER0, NCOUNTER = 192, 32     # per-slice arrival counters of the push side
WORK0 = 224                       # per-slice work counters of the slot sums (same count)
FLAG_WORDS = 256
RESET_BYTES = (FLAG_WORDS - RESET0) * 4


class _CudaBytes:
    """Adapter that lets torch wrap foreign device memory without copying."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None}


class SymmHeap:
    """Bump-allocated device heap that peers can address.

    ``group`` is a torch.distributed process group (or None for a single process).  The handle
    exchange uses ``all_gather_object`` on it, so it works over NCCL or Gloo groups alike.
    """

    def __init__(self, nbytes: int, group=None, device: Optional[torch.device] = None):
        import torch.distributed as dist
        self.C = _native.load()
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        self.nbytes = int(nbytes)
        self.base, handle = self.C.symm_alloc(self.nbytes)
        self._bytes = torch.as_tensor(_CudaBytes(self.base, self.nbytes), device=self.device)
        self._top = 0
        self.rank, self.world = 0, 1
        self.peer_base: List[int] = [self.base]
        if group is not None or (dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1):
            self.rank = dist.get_rank(group)
            self.world = dist.get_world_size(group)
            handles = [None] * self.world
            dist.all_gather_object(handles, handle, group=group)
            self.peer_base = [self.base if r == self.rank else self.C.symm_open(handles[r])
                              for r in range(self.world)]
            dist.barrier(group=group)

    def alloc(self, nbytes: int, align: int = 1024) -> int:
        off = (self._top + align - 1) // align * align
        if off + nbytes > self.nbytes:
            raise MemoryError(f"symmetric heap exhausted: need {nbytes} at {off} of {self.nbytes}")
        self._top = off + nbytes
        return off

    def bytes_view(self, off: int, nbytes: int) -> torch.Tensor:
        return self._bytes[off:off + nbytes]

    def tensor(self, off: int, shape, dtype=torch.bfloat16) -> torch.Tensor:
        n = int(np.prod(shape)) * torch.empty((), dtype=dtype).element_size()
        return self._bytes[off:off + n].view(dtype).view(*shape)

    def empty(self, shape, dtype=torch.bfloat16) -> torch.Tensor:
        n = int(np.prod(shape)) * torch.empty((), dtype=dtype).element_size()
        return self.tensor(self.alloc(n), shape, dtype)

    def ptr(self, rank: int, off: int) -> int:
        return self.peer_base[rank] + off

    def offset_of(self, t: torch.Tensor) -> Optional[int]:
        """Heap offset of a tensor that lives in this heap, else None."""
        p = t.data_ptr()
        if self.base <= p < self.base + self.nbytes:
            return p - self.base
        return None


@dataclass
class Workspace:
    """Scratch memory of one rank for the fused kernels.  All fields are byte offsets that are
    valid in every rank's heap (see SymmHeap)."""
    heap: SymmHeap
    stage_a_bytes: int
    stage_b_bytes: int
    slot_bytes: int
    flags: int = 0
    stage_a: int = 0
    stage_b: int = 0
    slots: int = 0
    epoch: int = 0
    _jobs_cache: Dict = field(default_factory=dict)

    def __post_init__(self):
        h = self.heap
        self.flags = h.alloc(FLAG_WORDS * 4)
        h.bytes_view(self.flags, FLAG_WORDS * 4).zero_()
        self.stage_a = h.alloc(max(self.stage_a_bytes, 16))
        self.stage_b = h.alloc(max(self.stage_b_bytes, 16))
        self.slots = h.alloc(max(self.slot_bytes, 16))
        torch.cuda.synchronize()

    # pointers into this rank's or a peer's copy of the workspace
    def flag_ptr(self, rank: int, word: int) -> int:
        return self.heap.ptr(rank, self.flags + 4 * word)

    def local(self, off: int) -> int:
        return self.heap.base + off

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch


class World:
    """Resolves (rank, workspace offset) to a device pointer.  The real implementation adds the
    offset to the peer's heap base; tests can emulate several ranks on one GPU by giving each
    emulated rank its own Workspace on a private heap."""

    def __init__(self, workspaces: List[Workspace], my_rank: int, single_heap: bool):
        self.ws = workspaces
        self.my_rank = my_rank
        self.single_heap = single_heap

    @classmethod
    def real(cls, ws: Workspace):
        w = cls([ws], ws.heap.rank, True)
        return w

    @property
    def mine(self) -> Workspace:
        return self.ws[0] if self.single_heap else self.ws[self.my_rank]

    @property
    def size(self) -> int:
        return self.mine.heap.world if self.single_heap else len(self.ws)

    def ptr(self, rank: int, off: int) -> int:
        if self.single_heap:
            return self.ws[0].heap.ptr(rank, off)
        return self.ws[rank].heap.base + off

    def flag_ptr(self, rank: int, word: int) -> int:
        return self.ptr(rank, self.mine.flags + 4 * word)


class RowExchanger:
    """Host side of the in-kernel exchange of a few floats per row among the GPUs of one mesh row
    (LayerNorm statistics, cross-entropy max / sum-exp / target logit): the counterpart of the
    ``psum`` over the mesh columns at ShardedLayers.py:129-131, without a collective call.

    The producing kernel writes its rows' partial values into this GPU's slot on every GPU of the
    group and counts one arrival per CTA on every peer; the consuming kernel waits for the arrivals
    of all peers' CTAs and sums the slots.  Two slot / counter sets alternate from call to call: a
    peer can be at most one call ahead (its consumer of call k needs this GPU's producer of call
    k), so what it writes for call k + 1 never lands in the set this GPU still reads for call k.
    Every rank of the group must issue the same sequence of exchanges."""

    WIDTH = 4        # floats reserved per row and source (LayerNorm uses 2, cross-entropy 3)

    def __init__(self, heap: SymmHeap, group_ranks: List[int], my_index: int, max_rows: int,
                 timeout_ns: int = 20_000_000_000):
        self.heap, self.ranks, self.me, self.max_rows = heap, list(group_ranks), my_index, max_rows
        self.n = len(self.ranks)
        self.timeout_ns = timeout_ns
        self.stride = max_rows * self.WIDTH                       # floats per source
        self.set_bytes = self.n * self.stride * 4
        self.slots = heap.alloc(2 * self.set_bytes)
        self.counters = heap.alloc(64)
        heap.bytes_view(self.counters, 64).zero_()
        self.calls = 0
        self.arrived = [0, 0]                                     # cumulative targets per set
        torch.cuda.synchronize()

    def next(self, rows: int, producer_grid: int):
        """Descriptors (producer, consumer) of the next exchange of ``rows`` rows; the producing
        kernel runs ``producer_grid`` CTAs on every GPU of the group."""
        if rows > self.max_rows:
            raise ValueError(f"row exchange sized for {self.max_rows} rows, got {rows}")
        k = self.calls & 1
        self.calls += 1
        self.arrived[k] = (self.arrived[k] + (self.n - 1) * producer_grid) & 0xffffffff
        base = self.slots + k * self.set_bytes
        d = dict(n=self.n, me=self.me,
                 dst=[self.heap.ptr(q, base + self.me * self.stride * 4) for q in self.ranks],
                 slots=self.heap.base + base, stride=self.stride,
                 counter=[self.heap.ptr(q, self.counters + 4 * k) for q in self.ranks],
                 my_counter=self.heap.base + self.counters + 4 * k, target=self.arrived[k],
                 timeout_ns=self.timeout_ns, status=_native.status().dev)
        return d, d


JOB_DTYPE = np.dtype([("src", "<u8"), ("dst", "<u8"), ("rows", "<u4"), ("row_bytes", "<u4"),
                      ("sp", "<u8"), ("dp", "<u8")])
PUSH_DTYPE = np.dtype([("src", "<u8"), ("rows", "<u4"), ("row_bytes", "<u4"), ("sp", "<u8"), ("dp", "<u8"),
                       ("n_dst", "<u4"), ("src_sel", "<u4"), ("dst", "<u8", (8,))])
CHUNK_DTYPE = np.dtype([("job_begin", "<i4"), ("job_end", "<i4"), ("n_sig", "<u4"), ("target", "<u4"),
                        ("sig", "<u8", (8,))])


def upload_jobs(jobs: List[tuple], chunk_begin: List[int], device) -> tuple:
    """Pull jobs of the stand-alone P2P collectives: (src, dst, rows, row_bytes, sp, dp)."""
    arr = np.array(jobs, dtype=JOB_DTYPE)
    assert arr.dtype.itemsize == _native.load().COPY_JOB_BYTES
    jt = torch.from_numpy(arr.view(np.uint8).copy()).to(device)
    bt = torch.tensor(chunk_begin, dtype=torch.int32, device=device)
    return jt, bt


def upload_push_plan(jobs: List[tuple], chunks: List[tuple], device) -> tuple:
    """Gather plan of the fused kernel.
    jobs:   (src_sel, src_offset, rows, row_bytes, src_pitch, dst_pitch, [dst pointers])
    chunks: (job_begin, job_end, [flag pointers], target)"""
    C = _native.load()
    ja = np.zeros(len(jobs), dtype=PUSH_DTYPE)
    for i, (sel, src, rows, rb, sp, dp, dsts) in enumerate(jobs):
        ja[i]["src"], ja[i]["rows"], ja[i]["row_bytes"], ja[i]["sp"], ja[i]["dp"] = src, rows, rb, sp, dp
        ja[i]["src_sel"] = sel
        ja[i]["n_dst"] = len(dsts)
        ja[i]["dst"][:len(dsts)] = dsts
    ca = np.zeros(len(chunks), dtype=CHUNK_DTYPE)
    for i, (jb, je, sigs, target) in enumerate(chunks):
        ca[i]["job_begin"], ca[i]["job_end"], ca[i]["n_sig"], ca[i]["target"] = jb, je, len(sigs), target
        ca[i]["sig"][:len(sigs)] = sigs
    assert ja.dtype.itemsize == C.PUSH_JOB_BYTES and ca.dtype.itemsize == C.CHUNK_DESC_BYTES
    jt = torch.from_numpy(ja.view(np.uint8).copy()).to(device)
    ct = torch.from_numpy(ca.view(np.uint8).copy()).to(device)
    return jt, ct
