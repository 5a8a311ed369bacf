#!/usr/bin/env python
"""One fused LS or RS case on ONE GPU for profiling the fused kernel's tile and reduce phases.

The ranks of a mesh axis are emulated one after another on the same device (every emulated rank has
its own heap and workspace, "peer" pointers point into the other emulated ranks' buffers, the
cross-GPU barriers are off), and a dataflow runs in phases over all emulated ranks, so no launch ever
waits for a kernel that is not running.  The phase 'gemm' is the full tile loop with the push
epilogue (all pushes land in local HBM), 'reduce' the slot sums; the phases are timed separately
and compared with the plain GEMM of the same shape.

    python bench/fused_case.py ls 4 8192 1024 16384 [slices] [iters]   # LS over C=4: m, k_local, N
    python bench/fused_case.py rs 2 2048 16384 4096 [slices] [iters]   # RS over R=2: k_local, M, n
    python bench/fused_case.py os 4 8192 1024 4096 [slices] [iters]    # OS over C=4: m, k_local, n (gather of X)
    ncu --set full --clock-control none -k regex:sm100_gemm_kernel -s 8 -c 2 -o prof python bench/fused_case.py ls 4 4096 1024 8192 4 1
"""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from meshslice_b200 import _native  # noqa: E402
from meshslice_b200.ops.gemm import gemm, sm_count  # noqa: E402
from meshslice_b200.parallel import runtime as rt  # noqa: E402
from meshslice_b200.parallel.fused import FusedGemm, MeshCoord  # noqa: E402


def setup(R, C, stage_a, stage_b, slots):
    wss = []
    for _ in range(R * C):
        heap = rt.SymmHeap(stage_a + stage_b + slots + (1 << 20))
        wss.append(rt.Workspace(heap, stage_a, stage_b, slots))
    ops = {}
    for r in range(R):
        for c in range(C):
            mc = MeshCoord(R, C, r, c)
            ops[(r, c)] = FusedGemm(mc, rt.World(wss, mc.rank, single_heap=False), sm_count(),
                                    timeout_ns=300_000_000, use_barriers=False)
    return ops


def timeit(fn, iters):
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    which, n = sys.argv[1], int(sys.argv[2])
    d0, d1, d2 = (int(v) for v in sys.argv[3:6])
    slices = int(sys.argv[6]) if len(sys.argv) > 6 else 4
    iters = int(sys.argv[7]) if len(sys.argv) > 7 else 3
    res = dict(case=which, ranks=n, dims=[d0, d1, d2], slices=slices)
    if which == "ls":        # Y[m, N/C] = RS_col(X[m, kl] @ W[N, kl]^T), R = 1
        m, kl, N = d0, d1, d2
        nc = N // n
        ops = setup(1, n, 16, N * kl * 2, n * m * nc * 2)
        xs = {k: torch.randn(m, kl, device="cuda").bfloat16() for k in ops}
        wsd = {k: torch.randn(N, kl, device="cuda").bfloat16() for k in ops}
        outs = {k: torch.empty(m, nc, device="cuda", dtype=torch.bfloat16) for k in ops}
        run = lambda phase: [op.ls(xs[k], [wsd[k].data_ptr()], m, kl, N, outs[k], n_slices=slices, phase=phase,
                                   reset=False) for k, op in ops.items()]
        k0 = (0, 0)
        y = torch.empty(m, N, device="cuda", dtype=torch.bfloat16)
        plain = lambda: gemm(xs[k0], wsd[k0], "nt", out=y)
        ref = sum(xs[(0, c)].float() @ wsd[(0, c)].float().t()[:, :nc] for c in range(n))
        flops = 2.0 * m * kl * N
    elif which == "rs":      # Y[M/R, n] = RS_row(X[kr, M]^T @ W[kr, n]), C = 1
        kr, M, nn = d0, d1, d2
        mr = M // n
        ops = setup(n, 1, kr * M * 2, 16, n * mr * nn * 2)
        xs = {k: torch.randn(kr, M, device="cuda").bfloat16() for k in ops}
        wsd = {k: torch.randn(kr, nn, device="cuda").bfloat16() for k in ops}
        outs = {k: torch.empty(mr, nn, device="cuda", dtype=torch.bfloat16) for k in ops}
        run = lambda phase: [op.rs([xs[k].data_ptr()], wsd[k], kr, M, nn, outs[k], n_slices=slices, phase=phase,
                                   reset=False) for k, op in ops.items()]
        k0 = (0, 0)
        y = torch.empty(M, nn, device="cuda", dtype=torch.bfloat16)
        plain = lambda: gemm(xs[k0], wsd[k0], "tn", out=y)
        ref = sum(xs[(r, 0)].float().t()[:mr] @ wsd[(r, 0)].float() for r in range(n))
        flops = 2.0 * kr * M * nn
    elif which == "os":      # Y[m, n] = AG_col(X)[m, C * kl] @ W[C * kl, n], R = 1: the gather side
        m, kl, nn = d0, d1, d2
        Kd = n * kl
        ops = setup(1, n, m * Kd * 2, 16, 16)
        xs = {k: torch.randn(m, kl, device="cuda").bfloat16() for k in ops}
        wsd = {k: torch.randn(Kd, nn, device="cuda").bfloat16() for k in ops}
        outs = {k: torch.empty(m, nn, device="cuda", dtype=torch.bfloat16) for k in ops}
        run = lambda phase: [op.os([xs[(0, c)].data_ptr() for c in range(n)], [wsd[k].data_ptr()], m, kl, Kd, nn, outs[k],
                                   n_slices=slices, phase=phase, reset=False) for k, op in ops.items()]
        k0 = (0, 0)
        xg = torch.cat([xs[(0, c)] for c in range(n)], dim=1)
        y = torch.empty(m, nn, device="cuda", dtype=torch.bfloat16)
        plain = lambda: gemm(xg, wsd[k0], "nn", out=y)
        ref = xg.float() @ wsd[k0].float()
        flops = 2.0 * m * Kd * nn
    else:
        raise SystemExit("first argument: os, ls or rs")
    for op in ops.values():
        op._reset_flags(_native.stream_ptr())
    if which == "os":
        # gather-only launches: every emulated rank writes its shard into all n staging buffers
        res["comm_ms"] = timeit(lambda: run("comm"), iters) / len(ops)
        res["gather_gbs_written"] = n * m * kl * 2 / (res["comm_ms"] * 1e-3) / 1e9
        _native.check_status()
    for phase in (("gemm",) if which == "os" else ("gemm", "reduce")):
        res[phase + "_ms"] = timeit(lambda: run(phase), iters) / len(ops)
        _native.check_status()
    res["plain_gemm_ms"] = timeit(plain, iters)
    res["gemm_phase_tflops"] = flops / res["gemm_ms"] / 1e9
    res["rel_err"] = ((outs[(0, 0)].float() - ref).norm() / ref.norm()).item()
    print(json.dumps(res))


if __name__ == "__main__":
    main()
