"""Names of TensorParallel1D.py mapped to this package."""
from ..parallel.tensor_parallel_1d import (SPMDWang, createShardedMatrix, fsdp as FSDP,  # noqa: F401
                                           wang_1d_is as Wang_1DIS, wang_1d_os as Wang_1DOS,
                                           wang_dp_os as Wang_DPOS)


def main(argv=None):
    """Self-test of the 1-D algorithms on an emulated 1 x 4 mesh (the checks of
    TensorParallel1D.py:129-160): output-stationary, input-stationary (its transpose product) and
    the sharded-weight data-parallel product against dense matmuls; prints one boolean per check."""
    import torch

    from ..parallel.mesh import EmuMesh, ShardedTensor
    from ..parallel.tensor_parallel import allclose
    B, S, H, D = 4, 128, 48, 64
    n = 4
    mesh = EmuMesh(1, n)
    X = torch.arange(B * S * H * D, dtype=torch.float32).reshape(B * S, H * D) / (B * S * H * D)
    W = torch.arange(H * D * 4 * H * D, dtype=torch.float32).reshape(H * D, 4 * H * D) / (4 * H * D * H * D)
    Y = X @ W
    dX = Y @ W.t()
    cols = lambda t: ShardedTensor(mesh, {(0, c): t.chunk(n, dim=1)[c].contiguous() for c in range(n)})
    rows = lambda t: ShardedTensor(mesh, {(0, c): t.chunk(n, dim=0)[c].contiguous() for c in range(n)})
    tp = SPMDWang(mesh)
    Xtp, Wtp = cols(X), cols(W)
    Ytp = tp.OS(Xtp, Wtp)
    results = [allclose(Ytp, cols(Y))]
    results.append(allclose(tp.IS(Ytp, Wtp), cols(dX)))
    results.append(allclose(tp.DP(rows(X), Wtp), rows(Y)))
    for ok in results:
        print(ok)
    return 0 if all(results) else 1


if __name__ == "__main__":
    raise SystemExit(main())
