"""Host-side logic of the fused dataflows, checked without a GPU: the gather plans of all ranks
of a mesh must fill every destination's staging buffer exactly once, chunk by chunk, and the
flag targets / reduce targets must equal the number of arrivals the kernels produce."""
import numpy as np
import pytest

from meshslice_b200.parallel import fused as fz
from meshslice_b200.parallel import runtime as rt


class FakeWS:
    """Workspace with fake, non-overlapping 'addresses' per rank."""
    def __init__(self, rank):
        base = (rank + 1) << 40
        self.flags, self.stage_a, self.stage_b, self.slots = 0, 1 << 20, 1 << 34, 1 << 36
        self.stage_a_bytes = self.stage_b_bytes = self.slot_bytes = 1 << 33
        self.base, self.epoch = base, 0

    def local(self, off):
        return self.base + off

    def next_epoch(self):
        self.epoch += 1
        return self.epoch


class FakeWorld:
    def __init__(self, n, me):
        self.wss = [FakeWS(r) for r in range(n)]
        self.my_rank, self.size = me, n

    @property
    def mine(self):
        return self.wss[self.my_rank]

    def ptr(self, rank, off):
        return self.wss[rank].base + off

    def flag_ptr(self, rank, word):
        return self.ptr(rank, 4 * word)


def _capture(R, C, call):
    """Runs `call(fg, mesh_coord)` for every rank and returns {rank: (plan, launch dict)}."""
    out = {}
    for r in range(R):
        for c in range(C):
            mc = fz.MeshCoord(R, C, r, c)
            fg = fz.FusedGemm.__new__(fz.FusedGemm)
            fg.mesh, fg.world, fg.grid, fg.timeout_ns, fg.use_barriers = mc, FakeWorld(R * C, mc.rank), 148, 1, False
            fg._cache = {}
            fg.signals = 148 * 2      # two communication warps per CTA bump every chunk flag
            cap = {}
            fg._jobs = lambda key, builder, cap=cap: (cap.setdefault("plan", builder()),
                                                      type("T", (), {"data_ptr": lambda s: 1})(),
                                                      type("T", (), {"data_ptr": lambda s: 2})(),
                                                      len(cap["plan"][1]))[1:]
            fg._launch = lambda d, exit_barrier, phase="all", reset=True, cap=cap: cap.setdefault("d", d)
            fg._common = lambda out_, acc, stream: {}
            call(fg, mc)
            out[mc.rank] = cap
    return out


class FakeT:
    def __init__(self, ptr, stride0):
        self._p, self._s = ptr, stride0

    def data_ptr(self):
        return self._p

    def stride(self, i):
        return self._s


@pytest.fixture(autouse=True)
def _no_gpu(monkeypatch):
    monkeypatch.setattr(fz._native, "stream_ptr", lambda: 0)


def _coverage(caps, dst_rank, stage_off, total_bytes, fake_base):
    """Bytes written into one destination's staging buffer by all ranks, as a counter array."""
    cnt = np.zeros(total_bytes // 16, dtype=np.int32)
    lo = fake_base + stage_off
    for cap in caps.values():
        if "plan" not in cap:
            continue
        jobs, _ = cap["plan"]
        for sel, src, rows, rb, sp, dp, dsts in jobs:
            for dptr in dsts:
                if not (lo <= dptr < lo + total_bytes):
                    continue
                for r in range(rows):
                    a = (dptr - lo + r * dp) // 16
                    cnt[a:a + rb // 16] += 1
    return cnt


@pytest.mark.parametrize("mesh", [(2, 4), (4, 2), (1, 8), (8, 1), (2, 2)])
def test_os_plans_fill_both_staging_buffers_once(mesh):
    R, C = mesh
    m, Kd, n = 1024, 2048, 512
    kl, kr = Kd // C, Kd // R
    caps = _capture(R, C, lambda fg, mc: fg.os([10 ** 9] * C, [2 * 10 ** 9] * R, m, kl, kr, n, None, n_slices=4))
    for rank in range(R * C):
        base = (rank + 1) << 40
        if C > 1:
            assert (_coverage(caps, rank, 1 << 20, m * Kd * 2, base) == 1).all()
        if R > 1:
            assert (_coverage(caps, rank, 1 << 34, Kd * n * 2, base) == 1).all()
        d = caps[rank]["d"]
        assert d["K"] == Kd and d["M"] == m and d["N"] == n
        if C == 1:
            assert d["A"] == 10 ** 9 and "a_flag_mode" not in d
        if R == 1:
            assert d["B"] == 2 * 10 ** 9 and "b_flag_mode" not in d
    # flag targets: every communication warp of every contributing GPU bumps each chunk once;
    # W travels in column chunks (flags 0 .. nW-1), X in row slices (flags nW ..), first wanted first
    if R > 1 and C > 1:
        _, chunks = caps[0]["plan"]
        d = caps[0]["d"]
        nW = d["b_flag_count"]
        assert d["b_flag_mode"] == 4 and d["a_flag_base"] == nW and nW == 2 and d["b_nchunk"] == 1
        flag0 = ((0 + 1) << 40) + 4 * rt.CHUNK0
        order = [(ch[2][0] - flag0) // 4 for ch in chunks]        # flag index of each chunk, in travel order
        assert order == [0, nW] + list(range(1, nW)) + list(range(nW + 1, nW + d["n_slices"]))
        for ch, idx in zip(chunks, order):
            assert ch[3] == 296 * (R if idx < nW else C)
        # what a consumer waits for is per operand, whatever the chunk's place in the travel order:
        # the arrivals at every flag of rank 0 (all sources, 296 warps each) equal that operand's target
        arrivals = {}
        for cap in caps.values():
            for (_jb, _je, sigs, _t) in cap["plan"][1]:
                for sp in sigs:
                    if (sp >> 40) == 1:
                        f = ((sp & ((1 << 40) - 1)) // 4) - rt.CHUNK0
                        arrivals[f] = arrivals.get(f, 0) + 296
        assert d["b_flag_target"] == 296 * R and d["a_flag_target"] == 296 * C
        for f, got in arrivals.items():
            assert got == (d["b_flag_target"] if f < nW else d["a_flag_target"]), (f, got)


@pytest.mark.parametrize("mesh", [(2, 4), (4, 2), (2, 2)])
def test_ls_and_rs_plans(mesh):
    R, C = mesh
    m, kl, nr = 512, 256, 1024 * C          # LS: X [m, kl], W shard [nr, kl]
    N = nr * R
    nc = N // C
    caps = _capture(R, C, lambda fg, mc: fg.ls(FakeT(5, kl), [3 * 10 ** 9] * R, m, kl, nr, None, n_slices=4))
    for rank in range(R * C):
        assert (_coverage(caps, rank, 1 << 34, N * kl * 2, (rank + 1) << 40) == 1).all()
        d = caps[rank]["d"]
        S = d["n_slices"]
        assert (nr // 256) % S == 0 and (nc // 256) % S == 0
        # arrivals per slice at an owner: C senders x its column blocks in the slice x row tiles x 4 warps
        assert d["red_target"] == C * (nc // 256 // S) * (m // 128) * 4
        assert len(d["push_base"]) == C and d["push_rows"] == m
    kr, ml, n = 384, 512 * R, 512             # RS: X shard [kr, ml], W [kr, n]
    M = ml * C
    mr = M // R
    caps = _capture(R, C, lambda fg, mc: fg.rs([7 * 10 ** 9] * C, FakeT(6, n), kr, ml, n, None, n_slices=2, cyc=2))
    for rank in range(R * C):
        assert (_coverage(caps, rank, 1 << 20, kr * M * 2, (rank + 1) << 40) == 1).all()
        d = caps[rank]["d"]
        S, cyc = d["n_slices"], d["cyc"]
        assert (ml // 256) % (S * cyc) == 0 and (mr // 256) % (S * cyc) == 0
        assert d["red_target"] == R * (mr // 128 // S) * (n // 256) * 4


def test_shapes_that_break_the_tile_rules_are_rejected():
    caps = {}
    with pytest.raises(fz.FusedPlanError):
        _capture(2, 2, lambda fg, mc: fg.ls(FakeT(5, 64), [1] * 2, 100, 64, 256, None))
    with pytest.raises(fz.FusedPlanError):
        _capture(2, 2, lambda fg, mc: fg.rs([1] * 2, FakeT(6, 100), 64, 256, 100, None))
    assert fz.pick_slices(8, 4) == 4 and fz.pick_slices(6, 4) == 3 and fz.pick_slices(4, 4, 2) == 2


@pytest.mark.parametrize("mesh,order,sub", [((2, 4), "summa", 2), ((2, 4), "wang", 1), ((4, 2), "wang", 2),
                                            ((2, 2), "cannon", 2), ((1, 4), "summa", 1), ((4, 1), "wang", 1)])
def test_k_panel_plans(mesh, order, sub):
    """SUMMA / Wang / Cannon schedules of the OS product: every panel reaches every consumer once,
    every panel flag is bumped by exactly one source, and a consumer's first panel is the first
    thing its source sends."""
    R, C = mesh
    m, Kd, n = 512, 2048, 512
    kl, kr = Kd // C, Kd // R
    caps = _capture(R, C, lambda fg, mc: fg.os_kpanel([10 ** 9] * C, [2 * 10 ** 9] * R, m, kl, kr, n, None,
                                                       order=order, sub=sub))
    flag_hits = {}
    for rank, cap in caps.items():
        d = cap["d"]
        base = (rank + 1) << 40
        if C > 1:
            assert (_coverage(caps, rank, 1 << 20, m * Kd * 2, base) == 1).all()
            assert d["a_flag_mode"] == 3 and d["a_kpanel"] * 64 * sub == kl
        if R > 1:
            assert (_coverage(caps, rank, 1 << 34, Kd * n * 2, base) == 1).all()
            assert d["b_flag_mode"] == 3 and d["b_kpanel"] * 64 * sub == kr and d["b_flag_base"] == C * sub
        r, c = divmod(rank, C)
        start = {"summa": 0, "wang": c * kl, "cannon": ((r + c) % C) * kl}[order]
        assert d["k_rot"] == start // 64 and d["kp_target"] == 296
        if "plan" in cap:
            jobs, chunks = cap["plan"]
            assert len(jobs) == len(chunks) and all(ch[1] - ch[0] == 1 and ch[3] == 296 for ch in chunks)
            for ch in chunks:
                for f in ch[2]:
                    flag_hits[f] = flag_hits.get(f, 0) + 1
    # one source per (destination, panel) flag; C*sub X panels and R*sub W panels per destination
    assert all(v == 1 for v in flag_hits.values())
    per_dest = (C * sub if C > 1 else 0) + (R * sub if R > 1 else 0)
    assert len(flag_hits) == per_dest * R * C
    if order == "wang" and C > 1:
        # the first X chunk a source emits is the one its own consumer starts with (its own panel)
        for rank, cap in caps.items():
            jobs, chunks = cap["plan"]
            first_x = next(i for i, j in enumerate(jobs) if j[0] == 0)
            own_flag = ((rank + 1) << 40) + 4 * (rt.CHUNK0 + (rank % C) * sub)
            assert chunks[first_x][2] == [own_flag]


@pytest.mark.parametrize("mesh", [(2, 4), (4, 2)])
@pytest.mark.parametrize("model", [dict(d=4096, f=16384, mb=16), dict(d=12288, f=49152, mb=8)])
def test_every_linear_of_the_benchmark_models_has_a_fused_plan(mesh, model):
    """Forward, data-gradient and weight-gradient products of the four linears of a block
    (6.7B-shaped and 175B-width) on both 8-GPU meshes: no shape falls back to the generic
    formulation, and chunk flags / slice counters stay inside the flag block."""
    R, C = mesh
    d, f = model["d"], model["f"]
    m = model["mb"] // R * 2048 if model["mb"] >= R else 2048          # tokens per rank and micro-batch
    lin = [(d, 3 * d, "os"), (d, d, "ls"), (d, f, "os"), (f, d, "ls")]
    for i, o, df in lin:
        def run(fg, mc, i=i, o=o, df=df):
            X = FakeT(5, i // C)
            if df == "os":
                fg.os([10 ** 9] * C, [2 * 10 ** 9] * R, m, i // C, i // R, o // C, None, n_slices=4)      # y = x W
                fg.ls(FakeT(5, o // C), [3 * 10 ** 9] * R, m, o // C, i // R, None, n_slices=4)          # dx = dy W^T
                fg.rs([7 * 10 ** 9] * C, FakeT(6, o // C), m, i // C, o // C, None, n_slices=4)          # dW = x^T dy
            else:
                fg.ls(X, [3 * 10 ** 9] * R, m, i // C, o // R, None, n_slices=4)                          # y = x W^T
                fg.os([10 ** 9] * C, [2 * 10 ** 9] * R, m, o // C, o // R, i // C, None, n_slices=4)      # dx = dy W
                fg.rs([7 * 10 ** 9] * C, FakeT(6, i // C), m, o // C, i // C, None, n_slices=4)          # dW = dy^T x
        calls = []
        def capture_all(fg, mc):
            real_launch = fg._launch
            fg._launch = lambda d_, exit_barrier, phase="all", reset=True: calls.append(d_)
            run(fg, mc)
        _capture(R, C, capture_all)
        assert len(calls) == 3 * R * C
        for d_ in calls:
            assert d_.get("n_chunks", 0) <= rt.NCHUNK
            assert d_["n_slices"] <= rt.NCOUNTER
            for k in ("M", "N", "K"):
                assert d_[k] > 0


@pytest.mark.parametrize("mesh", [(2, 4), (4, 2), (2, 2)])
def test_debug_validation_accepts_real_plans_and_rejects_corrupted_ones(mesh):
    """The host-side bounds checks of the debug mode: every address of the OS / LS / RS / K-panel
    plans lies inside a workspace buffer; a buffer that is too small, a stray destination, a wrong
    counter pointer or a signal that is not a chunk flag are refused before any launch."""
    R, C = mesh
    m, kl, kr, n = 1024, 2048 // C, 2048 // R, 512
    calls = {
        "os": lambda fg, mc: fg.os([10 ** 9] * C, [2 * 10 ** 9] * R, m, kl, kr, n, None, n_slices=4),
        "ls": lambda fg, mc: fg.ls(FakeT(5, 256), [3 * 10 ** 9] * R, 512, 256, 1024 * C, None, n_slices=4),
        "rs": lambda fg, mc: fg.rs([7 * 10 ** 9] * C, FakeT(6, 512), 384, 512 * R, 512, None, n_slices=2, cyc=2),
        "kp": lambda fg, mc: fg.os_kpanel([10 ** 9] * C, [2 * 10 ** 9] * R, m, kl, kr, n, None, order="wang", sub=2),
    }
    for name, call in calls.items():
        caps = _capture(R, C, call)
        for rank, cap in caps.items():
            mc = fz.MeshCoord(R, C, *divmod(rank, C))
            fg = fz.FusedGemm.__new__(fz.FusedGemm)
            fg.mesh, fg.world = mc, FakeWorld(R * C, rank)
            if "plan" in cap:
                fg.validate_plan(*cap["plan"])
            fg.validate_launch(cap["d"])
            # the same plan against staging buffers that are too small
            small = FakeWorld(R * C, rank)
            for w in small.wss:
                w.stage_a_bytes = w.stage_b_bytes = 4096
                w.slot_bytes = 4096
            fg.world = small
            if "plan" in cap and cap["plan"][0]:
                with pytest.raises(fz.FusedPlanError):
                    fg.validate_plan(*cap["plan"])
            if cap["d"].get("push_n", 0):
                with pytest.raises(fz.FusedPlanError):
                    fg.validate_launch(cap["d"])
            fg.world = FakeWorld(R * C, rank)
            if "plan" in cap and cap["plan"][1] and cap["plan"][1][0][2]:
                jobs, chunks = cap["plan"]
                bad = [(chunks[0][0], chunks[0][1], [chunks[0][2][0] + 4 * 1000], chunks[0][3])] + list(chunks[1:])
                with pytest.raises(fz.FusedPlanError):
                    fg.validate_plan(jobs, bad)
            if cap["d"].get("push_n", 0):
                d = dict(cap["d"])
                d["push_counter"] = [p + 4 for p in d["push_counter"]]
                with pytest.raises(fz.FusedPlanError):
                    fg.validate_launch(d)


@pytest.mark.parametrize("mesh", [(2, 4), (4, 2), (2, 2), (1, 4), (4, 1)])
@pytest.mark.parametrize("slices", [1, 2, 4])
def test_tile_order_matches_the_gather_chunks_and_the_arrival_targets(mesh, slices):
    """The kernel's tile map (mirrored by fused.tile_schedule) against the plans: every tile is
    visited once; a tile of slice s only reads gathered blocks that chunk s delivers; the number
    of partial tiles an owner counts per slice equals the reduce target."""
    R, C = mesh
    BMc, BNc = 256, 256

    def blocks_of_chunks(plan, stage_off, unit_bytes, block_units):
        """{chunk index: set of block indices (in tile units) that the chunk writes at rank 0}"""
        jobs, chunks = plan
        lo = (1 << 40) + stage_off
        out = {}
        for (jb, je, sigs, _t) in chunks:
            ci = (sigs[0] & ((1 << 40) - 1)) // 4 - rt.CHUNK0      # the chunk's flag index
            got = set()
            for sel, src, rows, rb, sp, dp, dsts in jobs[jb:je]:
                for dptr in dsts:
                    if lo <= dptr < lo + (1 << 33):
                        if block_units == "rows":      # blocks of rows of `unit_bytes` each
                            first, span = (dptr - lo) // unit_bytes, rows
                        else:                          # blocks of bf16 columns inside a row of pitch dp
                            first, span = ((dptr - lo) % dp) // 2, rb // 2
                        got.update(range(first // 256, (first + span + 255) // 256))
            out[ci] = got
        return out

    # ---- OS: X row blocks, sliced along M (flags xbase + s); W column blocks in chunks (flags 0 .. nW-1)
    m, Kd, n = 2048, 1024, 512
    caps = _capture(R, C, lambda fg, mc: fg.os([10 ** 9] * C, [2 * 10 ** 9] * R, m, Kd // C, Kd // R, n, None,
                                               n_slices=slices))
    d = caps[0]["d"]
    sched = fz.tile_schedule(d)
    assert sorted((a, b) for a, b, _ in sched) == [(i, j) for i in range(m // BMc) for j in range(-(-n // BNc))]
    if R > 1:
        per_chunk = {}
        for cap in caps.values():
            for ci, blks in blocks_of_chunks(cap["plan"], 1 << 34, 0, "cols").items():
                if ci < d["b_flag_count"]:
                    per_chunk.setdefault(ci, set()).update(blks)
        assert d["b_flag_mode"] == 4
        for mb, nb_, s_ in sched:
            assert nb_ in per_chunk[nb_ // d["b_nchunk"]]
    if C > 1:
        xbase = d["a_flag_base"]
        # union over all source ranks of the row blocks that chunk xbase + s delivers to rank 0
        per_chunk = {}
        for cap in caps.values():
            for ci, blks in blocks_of_chunks(cap["plan"], 1 << 20, Kd * 2, "rows").items():
                if ci >= xbase:
                    per_chunk.setdefault(ci - xbase, set()).update(blks)
        for mb, nb_, s_ in sched:
            assert mb in per_chunk[s_]

    # ---- LS: output columns sliced, partial tiles pushed to C owners
    mm, kl, nr = 512, 256, 1024 * C
    N = nr * R
    caps = _capture(R, C, lambda fg, mc: fg.ls(FakeT(5, kl), [3 * 10 ** 9] * R, mm, kl, nr, None, n_slices=slices))
    for rank, cap in caps.items():
        d = cap["d"]
        sched = fz.tile_schedule(d)
        assert len(set((a, b) for a, b, _ in sched)) == len(sched) == (mm // BMc) * (N // BNc)
        if C > 1:
            nc = N // C
            counts = {}
            for mb, nb_, s_ in sched:
                owner = nb_ * BNc // nc
                counts[(owner, s_)] = counts.get((owner, s_), 0) + 2 * 4     # two CTAs x four epilogue warps
            # every owner gets the same number from every sender: target = C senders x that number
            assert all(v * C == d["red_target"] for v in counts.values())
            assert len(counts) == C * d["n_slices"]
            # ranks of one mesh row start their slices at different owners
            first_owner = sched[0][1] * BNc // nc
            assert first_owner == ((rank % C) + 1) % C

    # ---- RS: output rows sliced (cyclic blocks of cyc tiles), pushed to R owners
    kr, ml, nn = 384, 512 * R, 512
    caps = _capture(R, C, lambda fg, mc: fg.rs([7 * 10 ** 9] * C, FakeT(6, nn), kr, ml, nn, None, n_slices=slices, cyc=2))
    M = ml * C
    for rank, cap in caps.items():
        d = cap["d"]
        sched = fz.tile_schedule(d)
        assert len(set((a, b) for a, b, _ in sched)) == len(sched) == (M // BMc) * (nn // BNc)
        if C > 1:
            per_chunk = {}
            # X columns (= output row blocks) of slice s come with chunk s
            for src_rank, cap2 in caps.items():
                if src_rank // C != rank // C:
                    continue      # only the ranks of this mesh row feed this rank's staging buffer
                jobs, chunks = cap2["plan"]
                lo = ((rank + 1) << 40) + (1 << 20)
                for ci, (jb, je, _s, _t) in enumerate(chunks):
                    for sel, src, rows, rb, sp, dp, dsts in jobs[jb:je]:
                        for dptr in dsts:
                            if lo <= dptr < lo + (1 << 33):
                                col0 = ((dptr - lo) % dp) // 2
                                per_chunk.setdefault(ci, set()).update(range(col0 // 256, (col0 + rb // 2) // 256))
            for mb, nb_, s_ in sched:
                assert mb in per_chunk[s_]
        if R > 1:
            mr = M // R
            counts = {}
            for mb, nb_, s_ in sched:
                counts[(mb * BMc // mr, s_)] = counts.get((mb * BMc // mr, s_), 0) + 8
            assert all(v * R == d["red_target"] for v in counts.values())


def _fg_with_flags(words):
    """A FusedGemm whose workspace flag block is a CPU tensor (what verify_flags reads after a launch)."""
    import torch
    flags = torch.zeros(rt.FLAG_WORDS, dtype=torch.int32)
    for k, v in words.items():
        flags[k] = v
    heap = type("H", (), {"bytes_view": lambda self, off, n: flags.view(torch.uint8)[off:off + n]})()
    ws = type("W", (), {"heap": heap, "flags": 0})()
    fg = fz.FusedGemm.__new__(fz.FusedGemm)
    fg.world = type("World", (), {"mine": ws})()
    return fg


def test_verify_flags_accepts_complete_flags_and_names_the_first_bad_one():
    last = dict(phase="all", K=512, n_slices=3, a_flag_mode=1, a_flag_base=2, a_flag_target=592,
                b_flag_mode=4, b_flag_base=0, b_flag_count=2, b_flag_target=1184, red_n=4, red_target=64)
    good = {rt.CHUNK0 + 0: 1184, rt.CHUNK0 + 1: 1184, rt.CHUNK0 + 2: 592, rt.CHUNK0 + 3: 592, rt.CHUNK0 + 4: 592,
            rt.COUNTER0 + 0: 64, rt.COUNTER0 + 1: 64, rt.COUNTER0 + 2: 64}
    fg = _fg_with_flags(good)
    fg._last = last
    fg.verify_flags()
    # a sender that was not counted, a flag signalled twice, a slice whose tiles did not all arrive
    for word, value, text in ((rt.CHUNK0 + 3, 591, "flag 3 of operand A"), (rt.CHUNK0 + 1, 2368, "flag 1 of operand B"),
                              (rt.COUNTER0 + 2, 60, "arrival counter of slice 2")):
        fg = _fg_with_flags({**good, word: value})
        fg._last = last
        with pytest.raises(fz.FlagProtocolError, match=text):
            fg.verify_flags()
    # K panels: one flag per panel of the contraction dimension, all at the panel target
    fg = _fg_with_flags({rt.CHUNK0 + 4 + i: 296 for i in range(4)})
    fg._last = dict(phase="gemm", K=1024, a_flag_mode=3, a_flag_base=4, a_kpanel=4, kp_target=296)
    fg.verify_flags()
    fg._last["K"] = 1280          # a fifth panel whose flag is still zero
    with pytest.raises(fz.FlagProtocolError, match="flag 8 of operand A"):
        fg.verify_flags()
    # a gather-only launch waits for nothing
    fg._last = dict(phase="comm", a_flag_mode=1, a_flag_base=0, n_slices=2, a_flag_target=5)
    fg.verify_flags()


def test_read_trace_decodes_and_clears_the_per_cta_event_areas():
    import torch
    fg = fz.FusedGemm.__new__(fz.FusedGemm)
    fg.grid, fg._trace_cap = 3, 4
    buf = torch.zeros(3, 5, 4, dtype=torch.int64)
    t0 = (7 << 32) + 0xfffffff0          # a timer value whose low word has the top bit set
    buf[0, 0, 0] = 2
    buf[0, 1] = torch.tensor([(t0 + 50) & 0xffffffff, (t0 + 50) >> 32, 2, 11])
    buf[0, 2] = torch.tensor([(t0 + 90) & 0xffffffff, (t0 + 90) >> 32, 6, 1])
    buf[2, 0, 0] = 9                     # more events than the area holds: only the stored ones come back
    for i in range(4):
        buf[2, 1 + i] = torch.tensor([(t0 + 10 * i) & 0xffffffff, (t0 + 10 * i) >> 32, 4, i])
    # the device buffer holds the 32-bit words as int32: wrap the values above 2^31
    fg._trace = torch.where(buf >= (1 << 31), buf - (1 << 32), buf).to(torch.int32).reshape(-1)
    ev = fg.read_trace()
    assert [e["t_ns"] for e in ev] == [0, 10, 20, 30, 50, 90]
    assert ev[0] == dict(t_ns=0, cta=2, kind="chunk_sent", arg=0)
    assert ev[4] == dict(t_ns=50, cta=0, kind="tile_computed", arg=11) and ev[5]["kind"] == "sum_end"
    assert fg.read_trace() == []


@pytest.mark.parametrize("mesh", [(1, 2), (2, 1), (2, 2), (2, 4), (4, 2), (1, 8), (8, 1)])
@pytest.mark.parametrize("model", ["gpt3-6.7b", "gpt3-175b-width"])
def test_trainer_workspace_fits_every_product_of_the_model(mesh, model):
    """The staging and slot buffers that the trainer allocates (`workspace_bytes`) hold the gathered operands and
    the pushed partial tiles of every forward, data-gradient and weight-gradient product of the block's four
    linears and of the LM head, for the 6.7B-shaped model and the 175B-width stack on every mesh shape."""
    from meshslice_b200.models.gpt import GPTConfig
    from meshslice_b200.trainer import workspace_bytes
    R, C = mesh
    if model == "gpt3-6.7b":
        cfg, gb = GPTConfig(), 32
    else:
        cfg, gb = GPTConfig(n_layers=4, d_model=12288, n_heads=96, ffn=49152), 16
    mb = max(1, min(gb // R, 16 if model == "gpt3-6.7b" else 8))
    sa, sb, sl = workspace_bytes(cfg, mb, R, C)
    m = mb * cfg.seq
    d, f, V = cfg.d_model, cfg.ffn, cfg.vocab_padded
    lin = [(d, 3 * d, cfg.dataflows[0]), (d, d, cfg.dataflows[1]), (d, f, cfg.dataflows[2]), (f, d, cfg.dataflows[3]),
           (d, V, "os")]
    assert set(cfg.dataflows) <= {"os", "ls"}

    def sized_world(n, me):
        w = FakeWorld(n, me)
        for ws in w.wss:
            ws.stage_a_bytes, ws.stage_b_bytes, ws.slot_bytes = sa, sb, sl
        return w

    for i, o, df in lin:
        for r in range(R):
            for c in range(C):
                mc = fz.MeshCoord(R, C, r, c)
                fg = fz.FusedGemm.__new__(fz.FusedGemm)
                fg.mesh, fg.world, fg.grid, fg.timeout_ns, fg.use_barriers = mc, sized_world(R * C, mc.rank), 148, 1, False
                fg._cache, fg.signals = {}, 296
                fg._jobs = lambda key, builder: (builder(), type("T", (), {"data_ptr": lambda s: 1})(),
                                                 type("T", (), {"data_ptr": lambda s: 2})(), 1)[1:]
                launched = []
                fg._launch = lambda d_, exit_barrier, phase="all", reset=True: launched.append(d_)
                fg._common = lambda out_, acc, stream: {}
                if df == "os":
                    fg.os([10 ** 9] * C, [2 * 10 ** 9] * R, m, i // C, i // R, o // C, None, n_slices=4)
                    fg.ls(FakeT(5, o // C), [3 * 10 ** 9] * R, m, o // C, i // R, None, n_slices=4)
                    fg.rs([7 * 10 ** 9] * C, FakeT(6, o // C), m, i // C, o // C, None, n_slices=4)
                else:
                    fg.ls(FakeT(5, i // C), [3 * 10 ** 9] * R, m, i // C, o // R, None, n_slices=4)
                    fg.os([10 ** 9] * C, [2 * 10 ** 9] * R, m, o // C, o // R, i // C, None, n_slices=4)
                    fg.rs([7 * 10 ** 9] * C, FakeT(6, i // C), m, o // C, i // C, None, n_slices=4)
                assert len(launched) == 3
    # what the 175B-width stack asks of one GPU stays far below its memory
    assert sa + sb + sl < 24 << 30
