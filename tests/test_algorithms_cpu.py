"""Every 2-D / 1-D GeMM algorithm on an emulated CPU mesh against the dense fp32 product."""
import pytest
import torch

from meshslice_b200.parallel.mesh import EmuMesh
from meshslice_b200.parallel.tensor_parallel import SPMD, allclose, createMultihostMatrix, slice_indices
from meshslice_b200.parallel.tensor_parallel_1d import SPMDWang, createShardedMatrix


def _mats(M, Kd, N, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(M, Kd, generator=g), torch.randn(Kd, N, generator=g)


def _run(mesh, alg, K, B, X, W):
    spmd = SPMD(mesh, alg, blocksize=B)
    Y = spmd.OS(K)(mesh.shard(X), mesh.shard(W))
    Yd = X @ W
    # LS recovers X from (Y, W) only as a product: dX-like = Y @ W^T ; RS: dW-like = X^T @ Y
    dX = spmd.LS(K)(mesh.shard(Yd), mesh.shard(W))
    dW = spmd.RS(K)(mesh.shard(X), mesh.shard(Yd))
    return mesh.unshard(Y), mesh.unshard(dX), mesh.unshard(dW), Yd, Yd @ W.t(), X.t() @ Yd


def test_baseline_config1_meshslice_2x2_slices4():
    """A[1024,2048] @ B[2048,1024], fp32, 2x2 mesh, 4 slices, forward + dA + dB at rtol 1e-4."""
    mesh = EmuMesh(2, 2)
    X, W = _mats(1024, 2048, 1024)
    Y, dX, dW, Yd, dXd, dWd = _run(mesh, "meshslice", 4, 8, X, W)
    for got, ref in ((Y, Yd), (dX, dXd), (dW, dWd)):
        assert torch.allclose(got, ref, rtol=1e-4, atol=1e-4 * ref.abs().max().item())


@pytest.mark.parametrize("shape", [(2, 2), (4, 2), (2, 4), (1, 8), (8, 1), (4, 4), (1, 1)])
@pytest.mark.parametrize("K,B", [(1, 8), (2, 8), (4, 8), (8, 8), (2, 64)])
def test_meshslice_matches_dense_on_all_mesh_shapes(shape, K, B):
    R, C = shape
    mesh = EmuMesh(R, C)
    unit = K * B * 8
    X, W = _mats(unit, unit * 2, unit, seed=R * 10 + C)
    Y, dX, dW, Yd, dXd, dWd = _run(mesh, "meshslice", K, B, X, W)
    for got, ref in ((Y, Yd), (dX, dXd), (dW, dWd)):
        assert torch.allclose(got, ref, rtol=1e-4, atol=1e-4 * ref.abs().max().item())


@pytest.mark.parametrize("alg,shape", [("collective", (4, 2)), ("collective", (2, 4)), ("wang", (4, 4)),
                                       ("wang", (4, 2)), ("wang", (2, 4)), ("cannon", (4, 4)),
                                       ("cannon", (2, 2)), ("summa", (2, 4)), ("summa", (4, 2)),
                                       ("summa", (4, 4)), ("meshflow", (4, 4))])
def test_baseline_algorithms_match_dense(alg, shape):
    """The reference's own self-test shapes (TensorParallel.py:427: B,S,H,D = 4,128,48,64)."""
    mesh = EmuMesh(*shape)
    B_, S, H, D = 4, 128, 48, 64
    g = torch.Generator().manual_seed(1)
    X = torch.randn(B_ * S, H * D // 4, generator=g) / 8
    W = torch.randn(H * D // 4, H * D, generator=g) / 8
    Y, dX, dW, Yd, dXd, dWd = _run(mesh, alg, 4, 8, X, W)
    for got, ref in ((Y, Yd), (dX, dXd), (dW, dWd)):
        assert torch.allclose(got, ref, rtol=1e-3, atol=1e-3 * ref.abs().max().item())


def test_cannon_rejects_non_square_mesh():
    with pytest.raises(ValueError):
        SPMD(EmuMesh(2, 4), "cannon")


def test_meshslice_equals_collective_on_non_square_mesh_notebook_shapes():
    """MeshFlowCPU.ipynb: 4x2 mesh, B, I, O = 512, 256, 1024."""
    mesh = EmuMesh(4, 2)
    X, W = _mats(512, 256, 1024, seed=5)
    a = SPMD(mesh, "meshslice").OS(4)(mesh.shard(X), mesh.shard(W))
    b = SPMD(mesh, "collective").OS()(mesh.shard(X), mesh.shard(W))
    assert allclose(a, b, atol=1e-4, rtol=1e-4)


def test_slices_are_block_cyclic_and_line_up_across_mesh_axes():
    """Slice i of the col-gathered X and of the row-gathered W cover the same ordered k set."""
    Kd, R, C, K, B = 1536, 2, 4, 4, 8
    for i in range(K):
        xs = torch.cat([c * (Kd // C) + slice_indices(Kd // C, K, B, i) for c in range(C)])
        ws = torch.cat([r * (Kd // R) + slice_indices(Kd // R, K, B, i) for r in range(R)])
        assert torch.equal(xs, ws)
        assert torch.equal(xs, torch.arange(Kd)[(torch.arange(Kd) // B) % K == i])
    allk = torch.cat([slice_indices(64, 4, 8, i) for i in range(4)]).sort().values
    assert torch.equal(allk, torch.arange(64))


def test_meshslice_rejects_indivisible_slicing():
    mesh = EmuMesh(2, 2)
    X, W = _mats(64, 48, 64)
    with pytest.raises(ValueError):
        SPMD(mesh, "meshslice").OS(4)(mesh.shard(X), mesh.shard(W))


def test_create_multihost_matrix_is_deterministic_per_coordinate():
    mesh = EmuMesh(2, 2)
    a = createMultihostMatrix(mesh, (64, 64), dtype=torch.float32, seed=3)
    b = createMultihostMatrix(mesh, (64, 64), dtype=torch.float32, seed=3)
    assert allclose(a, b, 0, 0)
    assert not torch.equal(a.shards[(0, 0)], a.shards[(0, 1)])


def test_1d_algorithms():
    """TensorParallel1D.py:129-160: OS, IS, FSDP and the DP-OS variant on 4 devices."""
    mesh = EmuMesh(1, 4)
    g = torch.Generator().manual_seed(0)
    Bt, I, O = 64, 128, 256
    X = torch.randn(Bt, I, generator=g)
    W = torch.randn(I, O, generator=g)
    sp = SPMDWang(mesh)
    Xs = mesh.shard_cols(X)
    Ws = mesh.shard_cols(W)
    Y = sp.OS(Xs, Ws)
    assert torch.allclose(torch.cat([Y.shards[(0, c)] for c in range(4)], 1), X @ W, atol=1e-3, rtol=1e-4)
    # IS: X [B, O/n] sharded on the contraction, W [I, O/n] -> X @ W^T  [B, I] sharded on columns
    Yfull = X @ W
    dX = sp.IS(mesh.shard_cols(Yfull), Ws)
    assert torch.allclose(torch.cat([dX.shards[(0, c)] for c in range(4)], 1), Yfull @ W.t(), atol=1e-2, rtol=1e-4)
    from meshslice_b200.parallel.mesh import ShardedTensor
    Xrows = ShardedTensor(mesh, {(0, c): X.chunk(4, 0)[c] for c in range(4)})
    Yd = sp.DP(Xrows, Ws)
    assert torch.allclose(torch.cat([Yd.shards[(0, c)] for c in range(4)], 0), X @ W, atol=1e-3, rtol=1e-4)
    Wrows = ShardedTensor(mesh, {(0, c): W.chunk(4, 0)[c] for c in range(4)})
    Y2 = sp.DPOS(Xrows, Wrows)
    assert torch.allclose(torch.cat([Y2.shards[(0, c)] for c in range(4)], 0), X @ W, atol=1e-3, rtol=1e-4)
    s = createShardedMatrix(mesh, (8, 16), dtype=torch.float32)
    assert s.shards[(0, 0)].shape == (8, 4)
