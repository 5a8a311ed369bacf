"""Names of TensorParallel.py mapped to this package."""
from ..parallel.mesh import DistMesh, EmuMesh, ShardedTensor  # noqa: F401
from ..parallel.tensor_parallel import (SPMD, allclose, createMultihostMatrix,  # noqa: F401
                                        cannon_ls as Cannon_LS, cannon_os as Cannon_OS, cannon_rs as Cannon_RS,
                                        collective_ls as Collective_LS, collective_os as Collective_OS,
                                        collective_rs as Collective_RS, meshslice_ls as MeshFlow_LS,
                                        meshslice_os as MeshFlow_OS, meshslice_rs as MeshFlow_RS,
                                        wang_ls as Wang_LS, wang_os as Wang_OS, wang_rs as Wang_RS)


def main(argv=None):
    """Self-test of one algorithm against the collective formulation on an emulated 4 x 4 mesh
    (the check of TensorParallel.py:425-457): ``python -m meshslice_b200.compat.TensorParallel wang``
    prints three booleans, one per dataflow (OS, LS, RS)."""
    import sys

    import torch
    alg = (argv if argv is not None else sys.argv[1:] or ["meshflow"])[0]
    B, S, H, D = 4, 128, 48, 64
    mesh = EmuMesh(4, 4)
    X = torch.arange(B * S * H * D, dtype=torch.float32).reshape(B * S, H * D) / (B * S * H * D)
    W = torch.arange(H * D * 4 * H * D, dtype=torch.float32).reshape(H * D, 4 * H * D) / (4 * H * D * H * D)
    Xo, Wo = mesh.shard(X), mesh.shard(W)
    mine, ref = SPMD(mesh, alg), SPMD(mesh, "collective")
    Yo = mine.OS()(Xo, Wo)
    results = [allclose(Yo, ref.OS()(Xo, Wo))]
    results.append(allclose(mine.LS()(Yo, Wo), ref.LS()(Yo, Wo)))      # dX = Y W^T
    results.append(allclose(mine.RS()(Xo, Yo), ref.RS()(Xo, Yo)))      # dW = X^T Y
    for ok in results:
        print(ok)
    return 0 if all(results) else 1


if __name__ == "__main__":
    raise SystemExit(main())
