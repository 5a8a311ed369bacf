"""Fused gather / push paths of the GEMM kernel on ONE GPU.

Several mesh ranks are emulated one after another: every emulated rank has its own heap and
workspace on the same device, "peer" pointers point into the other emulated ranks' buffers, and
the cross-GPU barriers are switched off.  Every dataflow runs in phases over all emulated ranks
(gather, then tiles, then slot sums), so no launch ever waits for a kernel that is not running.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(R, C, stage_a, stage_b, slots):
    from meshslice_b200.parallel import runtime as rt
    from meshslice_b200.parallel.fused import FusedGemm, MeshCoord
    from meshslice_b200.ops.gemm import sm_count
    wss = []
    for _ in range(R * C):
        heap = rt.SymmHeap(stage_a + stage_b + slots + (1 << 20))
        wss.append(rt.Workspace(heap, stage_a, stage_b, slots))
    ops = {}
    for r in range(R):
        for c in range(C):
            mc = MeshCoord(R, C, r, c)
            world = rt.World(wss, mc.rank, single_heap=False)
            ops[(r, c)] = FusedGemm(mc, world, sm_count(), timeout_ns=300_000_000, use_barriers=False)
    return ops, wss


def _close(out, ref, K):
    err = (out.float() - ref).abs().max().item()
    assert err < 0.03 * K ** 0.5 + 0.05, err
    assert ((out.float() - ref).norm() / ref.norm()).item() < 1.5e-2


@pytest.mark.parametrize("mesh,slices", [((2, 2), 2), ((1, 4), 1), ((4, 2), 4), ((2, 4), 2)])
def test_os_gathers_both_operands(mesh, slices):
    from meshslice_b200 import _native
    R, C = mesh
    M, Kd, N = 512 * R, 1024, 768 * C      # several W column chunks and X row slices on non-square meshes
    X = torch.randn(M, Kd, device="cuda").bfloat16()
    W = torch.randn(Kd, N, device="cuda").bfloat16()
    m, kl, kr, n = M // R, Kd // C, Kd // R, N // C
    xs = {(r, c): X[r * m:(r + 1) * m, c * kl:(c + 1) * kl].contiguous() for r in range(R) for c in range(C)}
    wsd = {(r, c): W[r * kr:(r + 1) * kr, c * n:(c + 1) * n].contiguous() for r in range(R) for c in range(C)}
    ops, _ = _setup(R, C, m * Kd * 2, Kd * n * 2, 16)
    ref = X.float() @ W.float()
    outs = {k: torch.empty(m, n, device="cuda", dtype=torch.bfloat16) for k in ops}
    for op in ops.values():
        op._reset_flags(_native.stream_ptr())
    for phase in ("comm", "gemm"):
        for (r, c), op in ops.items():
            op.os([xs[(r, cc)].data_ptr() for cc in range(C)], [wsd[(rr, c)].data_ptr() for rr in range(R)],
                  m, kl, kr, n, outs[(r, c)], n_slices=slices, phase=phase, reset=False)
            _native.check_status()
            if phase != "comm":
                op.verify_flags()
    for (r, c), out in outs.items():
        _close(out, ref[r * m:(r + 1) * m, c * n:(c + 1) * n], Kd)


@pytest.mark.parametrize("mesh,order,sub", [((2, 4), "summa", 2), ((2, 4), "wang", 1), ((2, 2), "cannon", 2),
                                            ((4, 2), "wang", 2), ((1, 2), "summa", 1)])
def test_os_k_panel_schedules(mesh, order, sub):
    """SUMMA / Wang / Cannon schedules: panels of the contraction dimension, consumed in the
    algorithm's order (rotated start of the contraction loop), give the dense product."""
    from meshslice_b200 import _native
    R, C = mesh
    M, Kd, N = 512 * R, 1024, 256 * C
    X = torch.randn(M, Kd, device="cuda").bfloat16()
    W = torch.randn(Kd, N, device="cuda").bfloat16()
    m, kl, kr, n = M // R, Kd // C, Kd // R, N // C
    xs = {(r, c): X[r * m:(r + 1) * m, c * kl:(c + 1) * kl].contiguous() for r in range(R) for c in range(C)}
    wsd = {(r, c): W[r * kr:(r + 1) * kr, c * n:(c + 1) * n].contiguous() for r in range(R) for c in range(C)}
    ops, _ = _setup(R, C, m * Kd * 2, Kd * n * 2, 16)
    ref = X.float() @ W.float()
    outs = {k: torch.empty(m, n, device="cuda", dtype=torch.bfloat16) for k in ops}
    for op in ops.values():
        op._reset_flags(_native.stream_ptr())
    for phase in ("comm", "gemm"):
        for (r, c), op in ops.items():
            op.os_kpanel([xs[(r, cc)].data_ptr() for cc in range(C)], [wsd[(rr, c)].data_ptr() for rr in range(R)],
                         m, kl, kr, n, outs[(r, c)], order=order, sub=sub, phase=phase, reset=False)
            _native.check_status()
            if phase != "comm":
                op.verify_flags()
    for (r, c), out in outs.items():
        _close(out, ref[r * m:(r + 1) * m, c * n:(c + 1) * n], Kd)


@pytest.mark.parametrize("mesh,slices", [((2, 2), 2), ((2, 4), 1)])
def test_ls_gathers_weights_pushes_over_row(mesh, slices):
    from meshslice_b200 import _native
    R, C = mesh
    M, Kd, N = 256 * R, 128 * C, 512 * R * C
    X = torch.randn(M, Kd, device="cuda").bfloat16()
    W = torch.randn(N, Kd, device="cuda").bfloat16()
    m, kl, nr, nc = M // R, Kd // C, N // R, N // C
    xs = {(r, c): X[r * m:(r + 1) * m, c * kl:(c + 1) * kl].contiguous() for r in range(R) for c in range(C)}
    wsd = {(r, c): W[r * nr:(r + 1) * nr, c * kl:(c + 1) * kl].contiguous() for r in range(R) for c in range(C)}
    ops, _ = _setup(R, C, 16, N * kl * 2, C * m * nc * 2)
    ref = X.float() @ W.float().t()
    outs = {k: torch.empty(m, nc, device="cuda", dtype=torch.bfloat16) for k in ops}
    for op in ops.values():
        op._reset_flags(_native.stream_ptr())
    for phase in ("comm", "gemm", "reduce"):
        for (r, c), op in ops.items():
            op.ls(xs[(r, c)], [wsd[(rr, c)].data_ptr() for rr in range(R)], m, kl, nr, outs[(r, c)],
                  n_slices=slices, phase=phase, reset=False)
            _native.check_status()
            if phase != "comm":
                op.verify_flags()
    for (r, c), out in outs.items():
        _close(out, ref[r * m:(r + 1) * m, c * nc:(c + 1) * nc], Kd)


def test_timeline_of_a_traced_ls_launch_and_identical_results():
    """The traced instantiation of the kernel records chunk, tile, push and slot-sum events for every emulated
    rank and computes bit-for-bit what the untraced one computes."""
    from meshslice_b200 import _native
    from meshslice_b200.utils.timing import fused_timeline_summary
    R, C, slices = 2, 2, 2
    M, Kd, N = 512 * R, 128 * C, 1024 * R * C
    X = torch.randn(M, Kd, device="cuda").bfloat16()
    W = torch.randn(N, Kd, device="cuda").bfloat16()
    m, kl, nr, nc = M // R, Kd // C, N // R, N // C
    xs = {(r, c): X[r * m:(r + 1) * m, c * kl:(c + 1) * kl].contiguous() for r in range(R) for c in range(C)}
    wsd = {(r, c): W[r * nr:(r + 1) * nr, c * kl:(c + 1) * kl].contiguous() for r in range(R) for c in range(C)}
    results = []
    for traced in (False, True):
        ops, _ = _setup(R, C, 16, N * kl * 2, C * m * nc * 2)
        outs = {k: torch.empty(m, nc, device="cuda", dtype=torch.bfloat16) for k in ops}
        for op in ops.values():
            op._reset_flags(_native.stream_ptr())
            if traced:
                op.enable_trace(256)
        for phase in ("comm", "gemm", "reduce"):
            for (r, c), op in ops.items():
                op.ls(xs[(r, c)], [wsd[(rr, c)].data_ptr() for rr in range(R)], m, kl, nr, outs[(r, c)],
                      n_slices=slices, phase=phase, reset=False)
                _native.check_status()
                if phase != "comm":
                    op.verify_flags()
        results.append(outs)
        if traced:
            tiles_per_rank = ((m + 255) // 256) * ((N + 255) // 256)
            for op in ops.values():
                ev = op.read_trace()
                kinds = {}
                for e in ev:
                    kinds[e["kind"]] = kinds.get(e["kind"], 0) + 1
                # one event per cluster tile from each CTA of the pair that computed it
                assert kinds.get("tile_computed", 0) == 2 * tiles_per_rank, kinds
                assert kinds.get("tile_pushed", 0) == 2 * tiles_per_rank, kinds
                assert kinds.get("operands_ready", 0) == 2 * tiles_per_rank, kinds
                assert kinds.get("chunk_sent", 0) > 0 and kinds.get("sum_begin", 0) == kinds.get("sum_end", 0) > 0
                assert all(a["t_ns"] <= b["t_ns"] for a, b in zip(ev, ev[1:]))
                s = fused_timeline_summary(ev)
                assert s["tile_computed"]["last_ns"] >= s["chunk_sent"]["first_ns"]
                assert op.read_trace() == []          # cleared
    for k in results[0]:
        assert torch.equal(results[0][k], results[1][k])


@pytest.mark.parametrize("mesh,slices,cyc", [((2, 2), 2, 1), ((2, 2), 1, 2), ((4, 2), 2, 2)])
def test_rs_gathers_inputs_pushes_over_column(mesh, slices, cyc):
    from meshslice_b200 import _native
    R, C = mesh
    Kd, M, N = 192 * R, 512 * R * C, 256 * C
    X = torch.randn(Kd, M, device="cuda").bfloat16()
    W = torch.randn(Kd, N, device="cuda").bfloat16()
    kr, ml, mr, n = Kd // R, M // C, M // R, N // C
    xs = {(r, c): X[r * kr:(r + 1) * kr, c * ml:(c + 1) * ml].contiguous() for r in range(R) for c in range(C)}
    wsd = {(r, c): W[r * kr:(r + 1) * kr, c * n:(c + 1) * n].contiguous() for r in range(R) for c in range(C)}
    ops, _ = _setup(R, C, kr * M * 2, 16, R * mr * n * 2)
    ref = X.float().t() @ W.float()
    outs = {k: torch.empty(mr, n, device="cuda", dtype=torch.bfloat16) for k in ops}
    for op in ops.values():
        op._reset_flags(_native.stream_ptr())
    for phase in ("comm", "gemm", "reduce"):
        for (r, c), op in ops.items():
            op.rs([xs[(r, cc)].data_ptr() for cc in range(C)], wsd[(r, c)], kr, ml, n, outs[(r, c)],
                  n_slices=slices, cyc=cyc, phase=phase, reset=False)
            _native.check_status()
            if phase != "comm":
                op.verify_flags()
    for (r, c), out in outs.items():
        _close(out, ref[r * mr:(r + 1) * mr, c * n:(c + 1) * n], Kd)


def test_bounded_wait_reports_timeout_instead_of_hanging():
    """A flag that nobody sets: the probe kernel gives up after its deadline and says so."""
    from meshslice_b200 import _native
    C = _native.load()
    flag = torch.zeros(1, device="cuda", dtype=torch.int32)
    st = torch.zeros(4, device="cuda", dtype=torch.int32)
    C.bounded_wait_probe(flag.data_ptr(), 1, 50_000_000, st.data_ptr(), _native.stream_ptr())
    torch.cuda.synchronize()
    assert st[0].item() == 1
    flag.fill_(5)
    st.zero_()
    C.bounded_wait_probe(flag.data_ptr(), 1, 50_000_000, st.data_ptr(), _native.stream_ptr())
    torch.cuda.synchronize()
    assert st[0].item() == 0
