"""Worker of the multi-GPU fused-kernel test: run under torchrun, one rank per GPU.
Compares the fused OS / LS / RS kernels (and the SUMMA / Wang / Cannon schedules of OS) with the dense fp32 product of the global operands."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl")
    from meshslice_b200 import _native
    from meshslice_b200.parallel.engine import FusedEngine
    from meshslice_b200.parallel.mesh import DistMesh

    R, C = [int(v) for v in os.environ.get("MESH", f"1x{world}").split("x")]
    slices = int(os.environ.get("SLICES", "2"))
    mesh = DistMesh(R, C)
    eng = FusedEngine(mesh, 64 << 20, 64 << 20, 64 << 20, timeout_ns=2_000_000_000, exchange_rows=4096)
    dev = torch.device("cuda")
    r, c = mesh.r, mesh.c
    g = torch.Generator(device="cpu").manual_seed(7)
    fails = []

    def close(name, out, ref, K):
        err = (out.float() - ref).abs().max().item()
        rel = ((out.float() - ref).norm() / ref.norm()).item()
        ok = err < 0.03 * K ** 0.5 + 0.05 and rel < 1.5e-2
        if not ok:
            fails.append(f"{name}: err {err} rel {rel}")

    for rep in range(3):
        # OS
        M, Kd, N = 512 * R, 1024 * 2, 512 * C
        X = torch.randn(M, Kd, generator=g).bfloat16().to(dev)
        W = torch.randn(Kd, N, generator=g).bfloat16().to(dev)
        m, kl, kr, n = M // R, Kd // C, Kd // R, N // C
        y = eng.os(X[r * m:(r + 1) * m, c * kl:(c + 1) * kl].contiguous(),
                   W[r * kr:(r + 1) * kr, c * n:(c + 1) * n].contiguous(), n_slices=slices)
        eng.check()
        close("os", y, (X.float() @ W.float())[r * m:(r + 1) * m, c * n:(c + 1) * n], Kd)
        # the same product on the K-panel schedules of the baseline algorithms
        xl = X[r * m:(r + 1) * m, c * kl:(c + 1) * kl].contiguous()
        wl = W[r * kr:(r + 1) * kr, c * n:(c + 1) * n].contiguous()
        for order in ("summa", "wang") + (("cannon",) if R == C else ()):
            y = eng.os_kpanel(xl, wl, order=order, sub=2)
            eng.check()
            close("os_" + order, y, (X.float() @ W.float())[r * m:(r + 1) * m, c * n:(c + 1) * n], Kd)
        # LS
        M, Kd, N = 256 * R, 256 * C, 512 * R * C
        X = torch.randn(M, Kd, generator=g).bfloat16().to(dev)
        W = torch.randn(N, Kd, generator=g).bfloat16().to(dev)
        m, kl, nr, nc = M // R, Kd // C, N // R, N // C
        y = eng.ls(X[r * m:(r + 1) * m, c * kl:(c + 1) * kl].contiguous(),
                   W[r * nr:(r + 1) * nr, c * kl:(c + 1) * kl].contiguous(), n_slices=slices)
        eng.check()
        close("ls", y, (X.float() @ W.float().t())[r * m:(r + 1) * m, c * nc:(c + 1) * nc], Kd)
        # RS
        Kd, M, N = 320 * R, 512 * R * C, 256 * C
        X = torch.randn(Kd, M, generator=g).bfloat16().to(dev)
        W = torch.randn(Kd, N, generator=g).bfloat16().to(dev)
        kr, ml, mr, n = Kd // R, M // C, M // R, N // C
        y = eng.rs(X[r * kr:(r + 1) * kr, c * ml:(c + 1) * ml].contiguous(),
                   W[r * kr:(r + 1) * kr, c * n:(c + 1) * n].contiguous(), n_slices=slices)
        eng.check()
        close("rs", y, (X.float().t() @ W.float())[r * mr:(r + 1) * mr, c * n:(c + 1) * n], Kd)

    t = torch.tensor([len(fails)], device=dev)
    dist.all_reduce(t)
    if fails:
        print(f"rank {rank} FAIL: {fails}", flush=True)
    if rank == 0:
        print("FUSED_MULTI_GPU_OK" if t.item() == 0 else "FUSED_MULTI_GPU_FAILED", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if t.item() == 0 else 1)


if __name__ == "__main__":
    main()
