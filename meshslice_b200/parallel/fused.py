"""Launch descriptions of the three fused MeshSlice dataflows on the tcgen05 GEMM kernel.

Global view used here (equivalent to the per-shard formulation of TensorParallel.py:153-214):

  OS   Y[m, n]   = X_g[m, :] @ W_g[:, n]    X_g = all-gather of X over the mesh row (concat on k),
                                            W_g = all-gather of W over the mesh column (concat on k)
  LS   Yp[m, :]  = X[m, :] @ W_g[:, :]^T    W_g = all-gather of W over the mesh column (concat on n),
                                            Y = reduce-scatter of Yp over the mesh row (split on n)
  RS   Yp[:, n]  = X_g[:, :]^T @ W[:, n]    X_g = all-gather of X over the mesh row (concat on m),
                                            Y = reduce-scatter of Yp over the mesh column (split on m)

"Mesh row" = the C devices that share a row index; "mesh column" = the R devices that share a
column index.  The slice count orders the work block-cyclically along the dimension whose data
moves (m for OS, n for LS, m for RS): slice s is gathered / pushed while slice s-1 is in the
tensor cores, and its flag is what the TMA producer of a tile waits for.  The result does not
depend on the slice count.
"""
from __future__ import annotations

import os

from dataclasses import dataclass
from typing import List, Optional

import torch

from .. import _native
from . import runtime as rt

BM, BN = 256, 256      # rows / columns of one cluster tile (two CTAs x 128 rows)
CTA_M = 128            # rows one CTA pushes per tile


@dataclass
class MeshCoord:
    R: int
    C: int
    r: int
    c: int

    @property
    def rank(self) -> int:
        return self.r * self.C + self.c

    def row_peers(self) -> List[int]:
        """Ranks of the mesh row (same r), indexed by column."""
        return [self.r * self.C + cc for cc in range(self.C)]

    def col_peers(self) -> List[int]:
        """Ranks of the mesh column (same c), indexed by row."""
        return [rr * self.C + self.c for rr in range(self.R)]


class FusedPlanError(ValueError):
    """The shapes do not meet the divisibility rules of the fused kernel."""


def _push_rotation(index: int, group: int, blocks_per_slice: int) -> int:
    """Block offset at which a rank starts every slice: the blocks of the *next* rank of its push
    group.  All ranks walk the owners in the same cyclic order but from different starting points,
    so at any time each owner receives from one rank, and a rank's own (local) blocks come last."""
    if os.environ.get("MSB_PUSH_ROT", "1") == "0":
        return 0
    return ((index + 1) % group) * (blocks_per_slice // group)


def tile_schedule(d: dict):
    """The order in which the fused kernel visits its 256 x 256 cluster tiles, as a list of
    (m_block, n_block, slice): a host-side mirror of the kernel's tile map (slice-major, raster
    groups of ``group`` blocks along the sliced dimension, block-cyclic slices of ``cyc`` blocks,
    rotation ``rot`` inside a slice).  Cluster c of n runs tiles c, c + n, c + 2n, ...  Used by tests
    and for reasoning about which chunk a tile waits for."""
    tiles_m = (d["M"] + BM - 1) // BM
    tiles_n = (d["N"] + BN - 1) // BN
    sd, S = d.get("slice_dim", 0), d.get("n_slices", 1)
    group, cyc, rot = max(1, d.get("group", 8)), max(1, d.get("cyc", 1)), d.get("rot", 0)
    tiles_s, tiles_o = (tiles_m, tiles_n) if sd == 0 else (tiles_n, tiles_m)
    nb = tiles_s // S
    if rot < 0 or rot >= nb:
        rot = 0
    out = []
    for t in range(tiles_m * tiles_n):
        s_, r = divmod(t, nb * tiles_o)
        g, rr = divmod(r, group * tiles_o)
        g0 = g * group
        o, w = divmod(rr, min(group, nb - g0))
        jj = g0 + w + rot
        if jj >= nb:
            jj -= nb
        cg = jj // cyc
        blk = (cg * S + s_) * cyc + (jj - cg * cyc)
        out.append((blk, o, s_) if sd == 0 else (o, blk, s_))
    return out


def pick_slices(n_blocks_per_part: int, want: int, cyc: int = 1) -> int:
    """Largest slice count <= want such that slices * cyc divides the blocks of every part."""
    s = max(1, min(want, n_blocks_per_part // cyc if cyc else 1))
    while s > 1 and n_blocks_per_part % (s * cyc) != 0:
        s -= 1
    return max(s, 1)


def _barrier_fields(world: rt.World, ranks: List[int], exit_barrier: bool, grid: int, timeout_ns: int):
    ws = world.mine
    n = world.size
    if n <= 1:
        return dict(n_ranks=0)
    epoch = ws.next_epoch()
    return dict(
        n_ranks=n, my_rank=world.my_rank,
        entry_flags=[world.flag_ptr(q, rt.ENTRY0) for q in range(n)],
        exit_flags=[world.flag_ptr(q, rt.EXIT0) for q in range(n)],
        epoch=epoch, go_flag=world.flag_ptr(world.my_rank, rt.GO),
        done_counter=world.flag_ptr(world.my_rank, rt.DONE), done_target=grid,
        exit_barrier=1 if exit_barrier else 0, timeout_ns=timeout_ns)


# event kinds of the fused kernel's timeline (TraceKind in csrc/gemm/sm100_gemm.h)
TRACE_KINDS = {1: "operands_ready", 2: "tile_computed", 3: "tile_pushed", 4: "chunk_sent", 5: "sum_begin",
               6: "sum_end"}


class FlagProtocolError(RuntimeError):
    """A flag or arrival counter of a finished fused launch does not stand at its target."""


class FusedGemm:
    """Builds and launches fused dataflows for one rank.

    ``world`` resolves peers' pointers (runtime.World).  ``x_ptrs`` / ``w_ptrs`` passed to the
    methods are the device pointers of every peer's shard (own shard included), indexed by the
    peer's position along the gathered mesh axis.
    """

    def __init__(self, mesh: MeshCoord, world: rt.World, grid: int, timeout_ns: int = 5_000_000_000,
                 use_barriers: bool = True, debug: Optional[bool] = None):
        # debug (or MSB_DEBUG_PLANS=1): every address that a plan hands to the kernel is checked on
        # the host against the workspace buffers before the launch (see validate_*)
        self.debug = (os.environ.get("MSB_DEBUG_PLANS", "0") == "1") if debug is None else debug
        self.mesh = mesh
        self.world = world
        self.grid = grid
        self.timeout_ns = timeout_ns
        self.use_barriers = use_barriers
        self.C = _native.load()
        # every communication warp of every CTA bumps a chunk's flag once per contributing GPU
        self.signals = grid * int(getattr(self.C, "AUX_WARPS", 1))
        self._cache = {}
        # staging buffers per epilogue warp of the push kernels (3 costs one pipeline stage)
        self.push_bufs = int(os.environ.get("MSB_PUSH_BUFS", "1"))
        # how partial tiles reach their owner: 0 = 2-D TMA tensor stores, 1 = ordinary 16-byte stores
        self.push_mode = int(os.environ.get("MSB_PUSH_MODE", "1"))
        self._trace = None          # timeline buffer of the next launches (enable_trace)
        self._trace_cap = 0

    # ------------------------------------------------------------------ helpers
    def _reset_flags(self, stream):
        ws = self.world.mine
        self.C.memset_zero(ws.local(ws.flags + 4 * rt.RESET0), rt.RESET_BYTES, stream)

    def _common(self, out, accumulate, stream):
        return dict(C=out.data_ptr(), ldc=out.stride(0), c_fp32=1 if out.dtype == torch.float32 else 0,
                    accumulate=1 if accumulate else 0, status=_native.status().dev, grid=self.grid,
                    stream=stream, timeout_ns=self.timeout_ns)

    # ------------------------------------------------------------------ plan validation
    def _region(self, ptr: int, nbytes: int, what: str):
        """(rank, buffer name) of the workspace buffer that holds [ptr, ptr + nbytes); raises
        FusedPlanError when the range is not inside one staging / slot buffer of one rank."""
        ws = self.world.mine
        for rank in range(self.world.size):
            for name, size in (("stage_a", ws.stage_a_bytes), ("stage_b", ws.stage_b_bytes), ("slots", ws.slot_bytes)):
                base = self.world.ptr(rank, getattr(ws, name))
                if base <= ptr and ptr + nbytes <= base + size:
                    return rank, name
        raise FusedPlanError(f"{what}: [{ptr:#x}, +{nbytes}) is outside every workspace buffer")

    def validate_plan(self, jobs, chunks):
        """Gather plan: every destination block lies inside a staging buffer, every signal is a chunk
        flag of some rank, chunk job ranges are ordered and inside the job list."""
        for i, (sel, src, rows, rb, sp, dp, dsts) in enumerate(jobs):
            if rows <= 0 or rb <= 0 or rb % 16 or src % 16 or sp % 16 or dp % 16 or sel not in (0, 1):
                raise FusedPlanError(f"job {i}: bad geometry (rows {rows}, row bytes {rb}, pitches {sp}/{dp})")
            if not 0 < len(dsts) <= 8:
                raise FusedPlanError(f"job {i}: {len(dsts)} destinations")
            for dptr in dsts:
                if dptr % 16:
                    raise FusedPlanError(f"job {i}: destination not 16-byte aligned")
                rank, name = self._region(dptr, (rows - 1) * dp + rb, f"job {i}")
                if name == "slots":
                    raise FusedPlanError(f"job {i}: gathers into the slot buffer of rank {rank}")
        ws = self.world.mine
        for i, (jb, je, sigs, target) in enumerate(chunks):
            if not 0 <= jb <= je <= len(jobs) or target <= 0 or len(sigs) > 8:
                raise FusedPlanError(f"chunk {i}: bad job range [{jb}, {je}) or target {target}")
            for sp_ in sigs:
                ok = False
                for rank in range(self.world.size):
                    word, rem = divmod(sp_ - self.world.ptr(rank, ws.flags), 4)
                    ok |= rem == 0 and rt.CHUNK0 <= word < rt.CHUNK0 + rt.NCHUNK
                if not ok:
                    raise FusedPlanError(f"chunk {i}: signal {sp_:#x} is not a chunk flag")

    def validate_launch(self, d):
        """Push / reduce side of a launch: owners' slot ranges, counters, slice and flag counts."""
        ws = self.world.mine
        if d.get("n_slices", 1) > rt.NCOUNTER:
            raise FusedPlanError("more slices than arrival counters")
        if d.get("n_chunks", 0) > rt.NCHUNK:
            raise FusedPlanError("more chunks than chunk flags")
        for mode, base, per in (("a_flag_mode", "a_flag_base", "a_kpanel"), ("b_flag_mode", "b_flag_base", "b_kpanel")):
            if d.get(mode, 0) == 3:
                kblocks = (d["K"] + 63) // 64
                if d.get(base, 0) + (kblocks + d[per] - 1) // d[per] > rt.NCHUNK:
                    raise FusedPlanError("K-panel flags beyond the flag block")
        if d.get("push_n", 0):
            extent = d["push_rows"] * d["push_ld"] * 2
            for o, (pb, pc) in enumerate(zip(d["push_base"], d["push_counter"])):
                rank, name = self._region(pb, extent, f"push slot of owner {o}")
                if name != "slots":
                    raise FusedPlanError(f"owner {o}: partial tiles pushed into {name}")
                if pc != self.world.flag_ptr(rank, rt.COUNTER0):
                    raise FusedPlanError(f"owner {o}: counter pointer is not rank {rank}'s counter block")
        if d.get("red_n", 0):
            if d["red_n"] * d["red_rows"] * d["red_ld"] * 2 > ws.slot_bytes or d["red_slots"] != ws.local(ws.slots):
                raise FusedPlanError("reduce phase reads beyond the slot buffer")

    def _jobs(self, key, builder):
        if key not in self._cache:
            jobs, chunks = builder()
            if self.debug:
                self.validate_plan(jobs, chunks)
            dev = torch.device("cuda", torch.cuda.current_device())
            self._cache[key] = rt.upload_push_plan(jobs, chunks, dev) + (len(chunks),)
        return self._cache[key]

    def _chunk_flag(self, rank: int, idx: int) -> int:
        return self.world.flag_ptr(rank, rt.CHUNK0 + idx)

    # ------------------------------------------------------------------ flag protocol
    def verify_flags(self) -> None:
        """Host-side check of the flag protocol after the last launch has finished: every chunk or panel flag
        that the tiles waited on stands exactly at its target (less: a sender was not counted; more: a flag was
        not cleared or a chunk was signalled twice) and so does every per-slice arrival counter of the slot
        sums.  Synchronises the device; meant for tests and debugging, not for the training loop."""
        d = getattr(self, "_last", None)
        if d is None or d.get("phase") not in ("all", "reduce", "gemm"):
            return
        ws = self.world.mine
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        words = ws.heap.bytes_view(ws.flags, rt.FLAG_WORDS * 4).view(torch.int32).cpu().numpy().astype("int64") & 0xffffffff
        bad = []

        def expect(word, target, what):
            if int(words[word]) != int(target):
                bad.append(f"{what}: {int(words[word])} != {int(target)}")

        kblocks = (d.get("K", 0) + 63) // 64
        for op in ("a", "b"):
            mode, base = d.get(f"{op}_flag_mode", 0), d.get(f"{op}_flag_base", 0)
            if mode == 1:
                idx, target = range(base, base + d.get("n_slices", 1)), d.get(f"{op}_flag_target", 0)
            elif mode in (2, 4):
                idx, target = range(base, base + d.get(f"{op}_flag_count", 0)), d.get(f"{op}_flag_target", 0)
            elif mode == 3:
                per = max(1, d.get(f"{op}_kpanel", 1))
                idx, target = range(base, base + (kblocks + per - 1) // per), d.get("kp_target", 0)
            else:
                continue
            if d.get("no_tiles", 0):
                continue          # a launch without tiles waits for nothing
            for i in idx:
                expect(rt.CHUNK0 + i, target, f"flag {i} of operand {op.upper()}")
        if d.get("red_n", 0):
            for sl in range(d.get("n_slices", 1)):
                expect(rt.COUNTER0 + sl, d.get("red_target", 0), f"arrival counter of slice {sl}")
        if bad:
            raise FlagProtocolError("; ".join(bad[:8]))

    # ------------------------------------------------------------------ timeline
    def enable_trace(self, events_per_cta: int = 512) -> None:
        """The following launches run the traced instantiation of the kernel: every CTA records when the
        gathered chunks of a tile had arrived, when the tile's accumulator was complete, when the partial tile
        had been pushed, when a communication warp had sent its share of a chunk and when the slot sums of a
        slice began and ended (``%globaltimer`` stamps; the per-slice overlap timeline).  ``read_trace``
        returns and clears them; ``disable_trace`` goes back to the untraced kernel."""
        self._trace_cap = int(events_per_cta)
        self._trace = torch.zeros(self.grid * (self._trace_cap + 1) * 4, dtype=torch.int32, device="cuda")

    def disable_trace(self) -> None:
        self._trace, self._trace_cap = None, 0

    def read_trace(self) -> List[dict]:
        """Events since the last call, sorted by time: dicts with ``t_ns`` (relative to the first event),
        ``cta``, ``kind`` (name) and ``arg`` (tile, chunk or slice index)."""
        if self._trace is None:
            return []
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        raw = self._trace.view(self.grid, self._trace_cap + 1, 4).cpu().numpy().astype("int64") & 0xffffffff
        self._trace.zero_()
        out = []
        for cta in range(self.grid):
            n = min(int(raw[cta, 0, 0]), self._trace_cap)
            for lo, hi, kind, arg in raw[cta, 1:1 + n]:
                out.append(dict(t_ns=int(lo) | (int(hi) << 32), cta=cta,
                                kind=TRACE_KINDS.get(int(kind), str(int(kind))), arg=int(arg)))
        out.sort(key=lambda e: e["t_ns"])
        t0 = out[0]["t_ns"] if out else 0
        for e in out:
            e["t_ns"] -= t0
        return out

    def _launch(self, d, exit_barrier, phase="all", reset=True):
        """phases 'comm' (gather only), 'gemm' (tiles only) and 'reduce' (slot sums only) split one
        launch in three; together with reset=False this lets a test run several emulated ranks
        one after another on one GPU without any launch waiting for a kernel that is not running."""
        if self.debug:
            self.validate_launch(d)
        if d.get("push_n", 0):
            d["push_bufs"] = self.push_bufs
            d["push_mode"] = self.push_mode
        if reset:
            self._reset_flags(d["stream"])
        if phase == "comm":          # only move the gathered operands
            d.update(no_tiles=1, red_n=0, push_n=0)
        elif phase == "gemm":        # tiles only: the chunks were filled by an earlier 'comm' launch
            d.update(red_n=0, skip_comm=1)
        elif phase == "reduce":
            d.update(no_tiles=1, n_chunks=0, push_n=0, a_flag_mode=0, b_flag_mode=0)
            if d.get("red_n", 0):
                # a reduce-only launch of the emulated-rank tests and benches: the arrival counters stay
                # as the tile phases left them, the work counters start from zero in a buffer of their own
                self._work = torch.zeros(rt.NCOUNTER, dtype=torch.int32, device="cuda")
                d["red_work"] = self._work.data_ptr()
        if self.use_barriers:
            d.update(_barrier_fields(self.world, [], exit_barrier, self.grid, self.timeout_ns))
        if self._trace is not None:
            d.update(trace=self._trace.data_ptr(), trace_cap=self._trace_cap)
        self._last = dict(d, phase=phase)
        self.C.gemm_run(d)

    # ------------------------------------------------------------------ OS
    def os(self, x_ptrs: List[int], w_ptrs: List[int], m: int, kl: int, kr: int, n: int, out,
           n_slices: int = 4, accumulate: bool = False, bias=None, act=None, pre_act=None,
           phase: str = "all", reset: bool = True):
        """Y[m, n] = concat_c(X_c)[m, C*kl] @ concat_r(W_r)[R*kr, n];  C*kl == R*kr."""
        mc, ws = self.mesh, self.world.mine
        Kd = mc.C * kl
        if Kd != mc.R * kr:
            raise FusedPlanError("OS: contraction sizes of X and W shards disagree")
        # a staging buffer is needed only for an operand that is gathered (a group of one reads in place)
        if kl % 8 or n % 8 or (mc.C > 1 and m * Kd * 2 > ws.stage_a_bytes) or (mc.R > 1 and Kd * n * 2 > ws.stage_b_bytes):
            raise FusedPlanError("OS: shard does not fit the staging buffers / alignment")
        tiles_m = (m + BM - 1) // BM
        S = pick_slices(tiles_m, n_slices)
        stream = _native.stream_ptr()
        xg, wg = ws.local(ws.stage_a), ws.local(ws.stage_b)

        rowp, colp = mc.row_peers(), mc.col_peers()
        x_mine, w_mine = x_ptrs[mc.c], w_ptrs[mc.r]

        gather_w, gather_x = mc.R > 1, mc.C > 1     # a group of one needs no copy at all
        # W travels in chunks of whole 256-column blocks, in the order in which the tile raster
        # reaches them, so the first tiles start after 1/nW of W (both operands are sliced and
        # pipelined, as in TensorParallel.py:159-172)
        tiles_n = (n + BN - 1) // BN
        nW = max(1, min(n_slices, tiles_n)) if gather_w else 0
        per = (tiles_n + nW - 1) // nW if gather_w else 1
        nW = (tiles_n + per - 1) // per if gather_w else 0
        xbase = nW                                  # index of the first X chunk

        def build():
            wjobs, xjobs = [], []
            for wc in range(nW):   # column block group wc of this rank's W shard -> every GPU of its mesh column
                col0 = wc * per * BN
                cols = min(n, col0 + per * BN) - col0
                wjobs.append([(1, col0 * 2, kr, cols * 2, n * 2, n * 2,
                               [self.world.ptr(q, ws.stage_b) + (mc.r * kr * n + col0) * 2 for q in colp])])
            for s in range(S if gather_x else 0):   # row blocks of this rank's X shard, block-cyclic
                js = []
                for blk in range(s, tiles_m, S):
                    row0 = blk * BM
                    rows = min(BM, m - row0)
                    js.append((0, row0 * kl * 2, rows, kl * 2, kl * 2, Kd * 2,
                               [self.world.ptr(q, ws.stage_a) + row0 * Kd * 2 + mc.c * kl * 2 for q in rowp]))
                xjobs.append(js)
            # order of travel = order of need: the first tiles want W chunk 0 and X slice 0, the first
            # sweep over the columns wants the rest of W, later slices of X are wanted last
            order = []
            if wjobs:
                order.append(("w", 0))
            if xjobs:
                order.append(("x", 0))
            order += [("w", i) for i in range(1, len(wjobs))] + [("x", i) for i in range(1, len(xjobs))]
            jobs, chunks = [], []
            for kind, i in order:
                jb = len(jobs)
                jobs += wjobs[i] if kind == "w" else xjobs[i]
                if kind == "w":
                    chunks.append((jb, len(jobs), [self._chunk_flag(q, i) for q in colp], self.signals * mc.R))
                else:
                    chunks.append((jb, len(jobs), [self._chunk_flag(q, xbase + i) for q in rowp], self.signals * mc.C))
            return jobs, chunks

        d = self._common(out, accumulate, stream)
        d.update(M=m, N=n, K=Kd, A=xg if gather_x else x_mine, B=wg if gather_w else w_mine, lda=Kd, ldb=n,
                 a_mn_major=0, b_mn_major=1, slice_dim=0, n_slices=S, cyc=1, group=8,
                 gather_src0=x_mine, gather_src1=w_mine)
        if gather_w or gather_x:
            jt, ct, n_chunks = self._jobs(("os", m, kl, kr, n, S, nW), build)
            d.update(jobs=jt.data_ptr(), chunks=ct.data_ptr(), n_chunks=n_chunks,
                     chunk_flags=ws.local(ws.flags + 4 * rt.CHUNK0))
            if gather_x:
                d.update(a_flag_mode=1, a_flag_base=xbase, a_flag_target=self.signals * mc.C)
            if gather_w:
                d.update(b_flag_mode=4, b_flag_base=0, b_flag_count=nW, b_nchunk=per, b_flag_target=self.signals * mc.R)
        if bias is not None:
            d["bias"] = bias.data_ptr()
        if act == "gelu":
            d["act"] = 1
            if pre_act is not None:
                d["C_pre"] = pre_act.data_ptr()
        self._launch(d, exit_barrier=False, phase=phase, reset=reset)
        return out

    # ------------------------------------------------------------------ OS, K-panel schedules
    def os_kpanel(self, x_ptrs: List[int], w_ptrs: List[int], m: int, kl: int, kr: int, n: int, out,
                  order: str = "summa", sub: int = 1, accumulate: bool = False,
                  phase: str = "all", reset: bool = True):
        """Y[m, n] = concat_c(X_c) @ concat_r(W_r) with the operands arriving in panels of the
        contraction dimension, the schedule of the SUMMA / Wang / Cannon baselines on one kernel:

        * ``summa``  every rank consumes the panels in the order 0, 1, 2, ...; the owner of a panel
          broadcasts it (one read of its shard, one store per peer).
        * ``wang``   a rank starts with the X panel it holds and walks the ring from there; a source
          serves its peers in the order in which they will need its panel.
        * ``cannon`` square meshes; rank (r, c) starts at panel (r + c) mod n, the skewed order of
          Cannon's algorithm, for both operands.

        ``sub`` splits every owner's panel into that many sub-panels (finer overlap).  On an NVSwitch
        fabric a "ring step" is a direct store to the peer that needs the panel next."""
        mc, ws = self.mesh, self.world.mine
        Kd = mc.C * kl
        if Kd != mc.R * kr:
            raise FusedPlanError("K-panel OS: contraction sizes of X and W shards disagree")
        if order not in ("summa", "wang", "cannon"):
            raise ValueError(f"unknown K-panel order {order!r}")
        if order == "cannon" and mc.R != mc.C:
            raise FusedPlanError("Cannon's schedule needs a square mesh")
        if (kl % 64 or kr % 64 or n % 8 or (mc.C > 1 and m * Kd * 2 > ws.stage_a_bytes)
                or (mc.R > 1 and Kd * n * 2 > ws.stage_b_bytes)):
            raise FusedPlanError("K-panel OS: shard does not fit the staging buffers / 64-wide k-blocks")
        sub = max(1, sub)
        while sub > 1 and (kl % (sub * 64) or kr % (sub * 64)):
            sub -= 1
        nA, nB = mc.C * sub, mc.R * sub
        if nA + nB > rt.NCHUNK:
            raise FusedPlanError("K-panel OS: too many panels")
        pa, pb = kl // sub, kr // sub
        stream = _native.stream_ptr()
        xg, wg = ws.local(ws.stage_a), ws.local(ws.stage_b)
        rowp, colp = mc.row_peers(), mc.col_peers()
        x_mine, w_mine = x_ptrs[mc.c], w_ptrs[mc.r]
        gather_w, gather_x = mc.R > 1, mc.C > 1

        def start(r, c):      # first contraction index that rank (r, c) consumes
            return {"summa": 0, "wang": c * kl, "cannon": ((r + c) % mc.C) * kl}[order]

        def build():
            recs = []         # (contraction distance at which the destinations need it, job, flags)
            if gather_x:
                groups = {}
                for cc, q in enumerate(rowp):
                    groups.setdefault((mc.c * kl - start(mc.r, cc)) % Kd, []).append(q)
                for t, dests in groups.items():
                    for s_ in range(sub):
                        job = (0, s_ * pa * 2, m, pa * 2, kl * 2, Kd * 2,
                               [self.world.ptr(q, ws.stage_a) + (mc.c * kl + s_ * pa) * 2 for q in dests])
                        recs.append((t + s_ * pa, job, [self._chunk_flag(q, mc.c * sub + s_) for q in dests]))
            if gather_w:
                groups = {}
                for rr, q in enumerate(colp):
                    groups.setdefault((mc.r * kr - start(rr, mc.c)) % Kd, []).append(q)
                for t, dests in groups.items():
                    for s_ in range(sub):
                        job = (1, s_ * pb * n * 2, pb, n * 2, n * 2, n * 2,
                               [self.world.ptr(q, ws.stage_b) + (mc.r * kr + s_ * pb) * n * 2 for q in dests])
                        recs.append((t + s_ * pb, job, [self._chunk_flag(q, nA + mc.r * sub + s_) for q in dests]))
            recs.sort(key=lambda rec: rec[0])
            jobs = [rec[1] for rec in recs]
            chunks = [(i, i + 1, rec[2], self.signals) for i, rec in enumerate(recs)]
            return jobs, chunks

        d = self._common(out, accumulate, stream)
        d.update(M=m, N=n, K=Kd, A=xg if gather_x else x_mine, B=wg if gather_w else w_mine, lda=Kd, ldb=n,
                 a_mn_major=0, b_mn_major=1, slice_dim=0, n_slices=1, cyc=1, group=8,
                 gather_src0=x_mine, gather_src1=w_mine, k_rot=start(mc.r, mc.c) // 64,
                 kp_target=self.signals)
        if gather_w or gather_x:
            jt, ct, n_chunks = self._jobs(("os_kpanel", order, m, kl, kr, n, sub), build)
            d.update(jobs=jt.data_ptr(), chunks=ct.data_ptr(), n_chunks=n_chunks,
                     chunk_flags=ws.local(ws.flags + 4 * rt.CHUNK0))
            if gather_x:
                d.update(a_flag_mode=3, a_flag_base=0, a_kpanel=pa // 64)
            if gather_w:
                d.update(b_flag_mode=3, b_flag_base=nA, b_kpanel=pb // 64)
        self._launch(d, exit_barrier=False, phase=phase, reset=reset)
        return out

    # ------------------------------------------------------------------ LS
    def ls(self, x, w_ptrs: List[int], m: int, kl: int, nr: int, out, n_slices: int = 4,
           accumulate: bool = False, phase: str = "all", reset: bool = True, rot_index: Optional[int] = None):
        """Y[m, N/C] = reduce-scatter over the mesh row of  X[m, kl] @ concat_r(W_r)[R*nr, kl]^T.

        ``rot_index`` selects at which owner's blocks this rank starts every slice: None = the rank
        after this one in its push group (MeshSlice; also the order in which Wang's rotating output
        accumulators visit the ranks), an explicit index i = the rank after i (Cannon's skew uses
        r + c), a negative value = no rotation (every rank walks the owners in the same order, the
        step order of SUMMA's reduce)."""
        mc, ws = self.mesh, self.world.mine
        N = mc.R * nr
        if N % mc.C:
            raise FusedPlanError("LS: output width not divisible by the mesh columns")
        nc = N // mc.C
        if nr % BN or nc % BN or m % BM or kl % 8:
            raise FusedPlanError("LS: shard sizes must be multiples of the 256x256 cluster tile")
        if N * kl * 2 > ws.stage_b_bytes or mc.C * m * nc * 2 > ws.slot_bytes:
            raise FusedPlanError("LS: staging / slot buffers too small")
        blocks_src, blocks_own = nr // BN, nc // BN
        import math
        S = pick_slices(math.gcd(blocks_src, blocks_own), n_slices)
        tiles_n, tiles_m = N // BN, m // BM
        stream = _native.stream_ptr()
        wg = ws.local(ws.stage_b)

        colp = mc.col_peers()
        w_mine = w_ptrs[mc.r]

        def build():
            jobs, chunks = [], []
            for s in range(S):     # n-blocks of this rank's W shard that belong to slice s
                jb = len(jobs)
                for blk in range(s, tiles_n, S):
                    row0 = blk * BN
                    if row0 // nr != mc.r:
                        continue
                    jobs.append((1, (row0 - mc.r * nr) * kl * 2, BN, kl * 2, kl * 2, kl * 2,
                                 [self.world.ptr(q, ws.stage_b) + row0 * kl * 2 for q in colp]))
                chunks.append((jb, len(jobs), [self._chunk_flag(q, s) for q in colp], self.signals * mc.R))
            return jobs, chunks

        peers = mc.row_peers()  # owners of the output column blocks, indexed by column
        d = self._common(out, accumulate, stream)
        gather_w = mc.R > 1     # a mesh column of one GPU already holds the whole W
        d.update(M=m, N=N, K=kl, A=x.data_ptr(), B=wg if gather_w else w_mine, lda=x.stride(0), ldb=kl,
                 a_mn_major=0, b_mn_major=0, slice_dim=1, n_slices=S, cyc=1, group=4, gather_src1=w_mine)
        if gather_w:
            jt, ct, n_chunks = self._jobs(("ls", m, kl, nr, S), build)
            d.update(jobs=jt.data_ptr(), chunks=ct.data_ptr(), n_chunks=n_chunks,
                     chunk_flags=ws.local(ws.flags + 4 * rt.CHUNK0), b_flag_mode=1, b_flag_base=0,
                     b_flag_target=self.signals * mc.R)
        if mc.C > 1:   # a mesh row of one GPU keeps its product: plain epilogue into `out`
            d.update(
                 push_n=mc.C, push_dim=1, push_extent=nc, push_ld=nc, push_rows=m,
                 push_base=[self.world.ptr(q, ws.slots) + mc.c * m * nc * 2 for q in peers],
                 push_counter=[self.world.flag_ptr(q, rt.COUNTER0) for q in peers],
                 red_n=mc.C, red_slots=ws.local(ws.slots), red_rows=m, red_cols=nc, red_ld=nc,
                 red_counter=ws.local(ws.flags + 4 * rt.COUNTER0), red_work=ws.local(ws.flags + 4 * rt.WORK0),
                 red_target=mc.C * (blocks_own // S) * (m // CTA_M) * 4, red_slice_dim=1,
                 rot=0 if (rot_index is not None and rot_index < 0) else
                 _push_rotation((mc.c if rot_index is None else rot_index) % mc.C, mc.C, tiles_n // S))
        self._launch(d, exit_barrier=False, phase=phase, reset=reset)
        return out

    # ------------------------------------------------------------------ RS
    def rs(self, x_ptrs: List[int], w, kr: int, ml: int, n: int, out, n_slices: int = 4,
           accumulate: bool = False, cyc: int = 2, phase: str = "all", reset: bool = True,
           rot_index: Optional[int] = None):
        """Y[M/R, n] = reduce-scatter over the mesh column of  concat_c(X_c)[kr, C*ml]^T @ W[kr, n].
        ``rot_index``: as in ``ls`` (along the mesh column)."""
        mc, ws = self.mesh, self.world.mine
        M = mc.C * ml
        if M % mc.R:
            raise FusedPlanError("RS: output height not divisible by the mesh rows")
        mr = M // mc.R
        if ml % BM or mr % BM or n % BN or kr % 8:
            raise FusedPlanError("RS: shard sizes must be multiples of the 256x256 cluster tile")
        if kr * M * 2 > ws.stage_a_bytes or mc.R * mr * n * 2 > ws.slot_bytes:
            raise FusedPlanError("RS: staging / slot buffers too small")
        import math
        g = math.gcd(ml // BM, mr // BM)
        while cyc > 1 and g % cyc:
            cyc //= 2
        S = pick_slices(g, n_slices, cyc)
        tiles_m, tiles_n = M // BM, n // BN
        stream = _native.stream_ptr()
        xg = ws.local(ws.stage_a)

        rowp = mc.row_peers()
        x_mine = x_ptrs[mc.c]

        def build():
            jobs, chunks = [], []
            ngroups = tiles_m // (S * cyc)
            for s in range(S):     # column groups of this rank's X shard that belong to slice s
                jb = len(jobs)
                for cg in range(ngroups):
                    col0 = (cg * S + s) * cyc * BM
                    if col0 // ml != mc.c:
                        continue
                    jobs.append((0, (col0 - mc.c * ml) * 2, kr, cyc * BM * 2, ml * 2, M * 2,
                                 [self.world.ptr(q, ws.stage_a) + col0 * 2 for q in rowp]))
                chunks.append((jb, len(jobs), [self._chunk_flag(q, s) for q in rowp], self.signals * mc.C))
            return jobs, chunks

        peers = mc.col_peers()  # owners of the output row blocks, indexed by row
        d = self._common(out, accumulate, stream)
        gather_x = mc.C > 1     # a mesh row of one GPU already holds the whole X
        d.update(M=M, N=n, K=kr, A=xg if gather_x else x_mine, B=w.data_ptr(), lda=M, ldb=w.stride(0),
                 a_mn_major=1, b_mn_major=1, slice_dim=0, n_slices=S, cyc=cyc, group=8, gather_src0=x_mine)
        if gather_x:
            jt, ct, n_chunks = self._jobs(("rs", kr, ml, n, S, cyc), build)
            d.update(jobs=jt.data_ptr(), chunks=ct.data_ptr(), n_chunks=n_chunks,
                     chunk_flags=ws.local(ws.flags + 4 * rt.CHUNK0), a_flag_mode=1, a_flag_base=0,
                     a_flag_target=self.signals * mc.C)
        if mc.R > 1:   # a mesh column of one GPU keeps its product: plain epilogue into `out`
            d.update(
                 push_n=mc.R, push_dim=0, push_extent=mr, push_ld=n, push_rows=mr,
                 push_base=[self.world.ptr(q, ws.slots) + mc.r * mr * n * 2 for q in peers],
                 push_counter=[self.world.flag_ptr(q, rt.COUNTER0) for q in peers],
                 red_n=mc.R, red_slots=ws.local(ws.slots), red_rows=mr, red_cols=n, red_ld=n,
                 red_counter=ws.local(ws.flags + 4 * rt.COUNTER0), red_work=ws.local(ws.flags + 4 * rt.WORK0),
                 red_target=mc.R * ((mr // BM) // S) * 2 * tiles_n * 4, red_slice_dim=0,
                 rot=0 if (rot_index is not None and rot_index < 0) else
                 _push_rotation((mc.r if rot_index is None else rot_index) % mc.R, mc.R, tiles_m // S))
        self._launch(d, exit_barrier=False, phase=phase, reset=reset)
        return out
