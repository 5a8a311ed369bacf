"""Device meshes and the collectives the 2-D GeMM algorithms are written against.

Two implementations of one small interface:

* ``EmuMesh`` keeps every shard of an R x C mesh in one process (a dict keyed by mesh
  coordinate) and implements the collectives by indexing.  It is the CPU oracle of this
  package, the counterpart of running the reference on
  ``--xla_force_host_platform_device_count`` CPU devices (TensorParallel.py:429-432).
* ``DistMesh`` is one rank of a ``torch.distributed`` job (NCCL on GPUs, Gloo on CPUs): it
  owns exactly one coordinate and maps the same collectives to all-gather / reduce-scatter /
  send-recv on the row and column process groups.  On GPUs this is the NCCL baseline that the
  fused kernels are compared with.

Axis names follow the reference: collectives "along 'col'" run among the C devices of one mesh
row (same row index), "along 'row'" among the R devices of one mesh column.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Tuple

import torch

Coord = Tuple[int, int]


class ShardedTensor:
    """The shards of one logical tensor that this process holds, keyed by mesh coordinate."""

    def __init__(self, mesh: "Mesh", shards: Dict[Coord, torch.Tensor]):
        self.mesh = mesh
        self.shards = shards

    def map(self, fn: Callable[[torch.Tensor], torch.Tensor]) -> "ShardedTensor":
        return ShardedTensor(self.mesh, {k: fn(v) for k, v in self.shards.items()})

    def local(self) -> torch.Tensor:
        """The single shard of a one-coordinate mesh (DistMesh)."""
        (v,) = self.shards.values()
        return v

    def __add__(self, other):
        return self.mesh.map(lambda r, c, a, b: a + b, self, other)

    @property
    def shape(self):
        return next(iter(self.shards.values())).shape

    @property
    def dtype(self):
        return next(iter(self.shards.values())).dtype


class Mesh:
    """Interface shared by EmuMesh and DistMesh."""

    R: int
    C: int
    axis_names = ("row", "col")

    @property
    def shape(self):
        return (self.R, self.C)

    def coords(self) -> List[Coord]:
        raise NotImplementedError

    def axis_size(self, axis: str) -> int:
        return self.C if axis == "col" else self.R

    def map(self, fn, *sts: ShardedTensor) -> ShardedTensor:
        """fn(r, c, *local_tensors) for every coordinate this process holds."""
        return ShardedTensor(self, {k: fn(k[0], k[1], *[s.shards[k] for s in sts]) for k in self.coords()})

    # -- data placement --------------------------------------------------------------------
    def shard(self, full: torch.Tensor) -> ShardedTensor:
        """Block-shards a 2-D tensor P(row, col): dim 0 over rows, dim 1 over columns."""
        d0, d1 = full.shape
        if d0 % self.R or d1 % self.C:
            raise ValueError(f"shape {tuple(full.shape)} not divisible by mesh {self.shape}")
        b0, b1 = d0 // self.R, d1 // self.C
        return ShardedTensor(self, {(r, c): full[r * b0:(r + 1) * b0, c * b1:(c + 1) * b1].contiguous()
                                    for (r, c) in self.coords()})

    def shard_cols(self, full: torch.Tensor) -> ShardedTensor:
        """P(None, col) for the last dim: replicated over rows."""
        n = full.shape[-1]
        b = n // self.C
        return ShardedTensor(self, {(r, c): full[..., c * b:(c + 1) * b].contiguous() for (r, c) in self.coords()})

    def unshard(self, st: ShardedTensor) -> torch.Tensor:
        raise NotImplementedError

    # -- collectives -------------------------------------------------------------------------
    def all_gather(self, st: ShardedTensor, axis: str, dim: int) -> ShardedTensor:
        raise NotImplementedError

    def reduce_scatter(self, st: ShardedTensor, axis: str, dim: int) -> ShardedTensor:
        raise NotImplementedError

    def all_reduce(self, st: ShardedTensor, axis: str, op: str = "sum") -> ShardedTensor:
        raise NotImplementedError

    def permute(self, st: ShardedTensor, axis: str, shift: int) -> ShardedTensor:
        """Ring shift: the shard of index i along ``axis`` moves to index (i + shift) % size."""
        raise NotImplementedError

    def broadcast(self, st: ShardedTensor, axis: str, src: int) -> ShardedTensor:
        """Every device receives the shard of the device with index ``src`` along ``axis``."""
        g = self.all_gather(st.map(lambda t: t.unsqueeze(0)), axis, 0)
        return g.map(lambda t: t[src])

    def transpose(self, st: ShardedTensor) -> ShardedTensor:
        """Global transpose of a P(row, col) matrix: [A, B] sharded (A/R, B/C) becomes [B, A] sharded
        (B/R, A/C).  This is the re-orientation of activations that an 'rs' layer asks for (the
        ``Transpose`` node of the reference's compute graph, Autotuner.py:304-337).  Generic form:
        gather the matrix along both axes and cut the own block; a mesh may do better."""
        rows = self.all_gather(st, "col", 1)
        full = self.all_gather(rows, "row", 0)
        out = {}
        for (r, c), f in full.shards.items():
            A, B = f.shape
            if B % self.R or A % self.C:
                raise ValueError(f"cannot transpose a {A} x {B} matrix on mesh {self.shape}")
            b0, a0 = B // self.R, A // self.C
            out[(r, c)] = f[c * a0:(c + 1) * a0, r * b0:(r + 1) * b0].t().contiguous()
        return ShardedTensor(self, out)

    def reduce_to(self, st: ShardedTensor, axis: str, dst: int) -> ShardedTensor:
        """Sum along ``axis``; only the device with index ``dst`` is required to use the result."""
        return self.all_reduce(st, axis)


class EmuMesh(Mesh):
    """All R x C shards live in this process."""

    def __init__(self, R: int, C: int):
        self.R, self.C = R, C

    def coords(self):
        return [(r, c) for r in range(self.R) for c in range(self.C)]

    def _peers(self, r, c, axis):
        return [(r, cc) for cc in range(self.C)] if axis == "col" else [(rr, c) for rr in range(self.R)]

    def _index(self, r, c, axis):
        return c if axis == "col" else r

    def unshard(self, st):
        rows = [torch.cat([st.shards[(r, c)] for c in range(self.C)], dim=1) for r in range(self.R)]
        return torch.cat(rows, dim=0)

    def all_gather(self, st, axis, dim):
        return ShardedTensor(self, {(r, c): torch.cat([st.shards[p] for p in self._peers(r, c, axis)], dim=dim)
                                    for (r, c) in self.coords()})

    def reduce_scatter(self, st, axis, dim):
        n = self.axis_size(axis)
        out = {}
        for (r, c) in self.coords():
            total = sum(st.shards[p] for p in self._peers(r, c, axis))
            out[(r, c)] = total.chunk(n, dim=dim)[self._index(r, c, axis)].contiguous()
        return ShardedTensor(self, out)

    def all_reduce(self, st, axis, op="sum"):
        out = {}
        for (r, c) in self.coords():
            ts = [st.shards[p] for p in self._peers(r, c, axis)]
            out[(r, c)] = sum(ts) if op == "sum" else torch.stack(ts).max(0).values
        return ShardedTensor(self, out)

    def permute(self, st, axis, shift):
        n = self.axis_size(axis)
        out = {}
        for (r, c) in self.coords():
            if axis == "col":
                out[(r, (c + shift) % n)] = st.shards[(r, c)]
            else:
                out[((r + shift) % n, c)] = st.shards[(r, c)]
        return ShardedTensor(self, out)


class DistMesh(Mesh):
    """One rank of a torch.distributed job arranged as an R x C mesh (rank = r * C + c)."""

    def __init__(self, R: int, C: int, group=None):
        import torch.distributed as dist
        self.dist = dist
        self.R, self.C = R, C
        self.world = dist.get_world_size(group)
        if R * C != self.world:
            raise ValueError(f"mesh {R}x{C} does not match world size {self.world}")
        self.rank = dist.get_rank(group)
        self.r, self.c = divmod(self.rank, C)
        self.group = group
        # every rank must create every group, in the same order
        self.col_groups = [dist.new_group([rr * C + cc for cc in range(C)]) for rr in range(R)]
        self.row_groups = [dist.new_group([rr * C + cc for rr in range(R)]) for cc in range(C)]

    def coords(self):
        return [(self.r, self.c)]

    def _group(self, axis):
        return self.col_groups[self.r] if axis == "col" else self.row_groups[self.c]

    def _ranks(self, axis):
        return ([self.r * self.C + cc for cc in range(self.C)] if axis == "col"
                else [rr * self.C + self.c for rr in range(self.R)])

    def _index(self, axis):
        return self.c if axis == "col" else self.r

    def unshard(self, st):
        t = st.local()
        rows = self.all_gather(st, "col", 1)
        full = self.all_gather(rows, "row", 0)
        return full.local()

    def all_gather(self, st, axis, dim):
        x = st.local().contiguous()
        n = self.axis_size(axis)
        if n == 1:
            return ShardedTensor(self, {(self.r, self.c): x})
        out = torch.empty((n,) + tuple(x.shape), dtype=x.dtype, device=x.device)
        if x.is_cuda:
            self.dist.all_gather_into_tensor(out, x, group=self._group(axis))
        else:   # Gloo has no flat all-gather
            self.dist.all_gather([out[i] for i in range(n)], x, group=self._group(axis))
        parts = [out[i] for i in range(n)]
        return ShardedTensor(self, {(self.r, self.c): torch.cat(parts, dim=dim) if dim != 0 else out.reshape(-1, *x.shape[1:])})

    def reduce_scatter(self, st, axis, dim):
        x = st.local()
        n = self.axis_size(axis)
        if n == 1:
            return ShardedTensor(self, {(self.r, self.c): x})
        if dim != 0:
            x = torch.stack(x.chunk(n, dim=dim), 0)
        else:
            x = x.reshape(n, x.shape[0] // n, *x.shape[1:])
        x = x.contiguous()
        if x.is_cuda:
            out = torch.empty(x.shape[1:], dtype=x.dtype, device=x.device)
            self.dist.reduce_scatter_tensor(out, x, group=self._group(axis))
        else:   # Gloo has no reduce-scatter: all-reduce and keep the own chunk
            self.dist.all_reduce(x, group=self._group(axis))
            out = x[self._index(axis)].clone()
        return ShardedTensor(self, {(self.r, self.c): out})

    def all_reduce(self, st, axis, op="sum"):
        x = st.local().clone()
        if self.axis_size(axis) > 1:
            self.dist.all_reduce(x, op=self.dist.ReduceOp.SUM if op == "sum" else self.dist.ReduceOp.MAX,
                                 group=self._group(axis))
        return ShardedTensor(self, {(self.r, self.c): x})

    def permute(self, st, axis, shift):
        x = st.local().contiguous()
        n = self.axis_size(axis)
        if n == 1 or shift % n == 0:
            return ShardedTensor(self, {(self.r, self.c): x})
        ranks = self._ranks(axis)
        i = self._index(axis)
        dst, src = ranks[(i + shift) % n], ranks[(i - shift) % n]
        out = torch.empty_like(x)
        ops = [self.dist.P2POp(self.dist.isend, x, dst), self.dist.P2POp(self.dist.irecv, out, src)]
        for w in self.dist.batch_isend_irecv(ops):
            w.wait()
        return ShardedTensor(self, {(self.r, self.c): out})
