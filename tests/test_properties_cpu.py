"""Property-based checks (hypothesis) of the algorithm level on emulated meshes: for random mesh
shapes, slice counts, block sizes and operand sizes every 2-D algorithm equals the dense product,
slices partition their index range, and the fused kernel's tile map is a permutation."""
import pytest
import torch

hyp = pytest.importorskip("hypothesis")
from hypothesis import given, settings, strategies as st  # noqa: E402

from meshslice_b200.parallel import fused as fz  # noqa: E402
from meshslice_b200.parallel import tensor_parallel as tp  # noqa: E402
from meshslice_b200.parallel.mesh import EmuMesh  # noqa: E402

MESHES = [(1, 2), (2, 1), (2, 2), (2, 3), (3, 2), (4, 2), (1, 4)]


@settings(max_examples=25, deadline=None)
@given(mesh=st.sampled_from(MESHES), K=st.sampled_from([1, 2, 3, 4]), B=st.sampled_from([1, 2, 4]),
       mi=st.integers(1, 3), ki=st.integers(1, 2), ni=st.integers(1, 2), seed=st.integers(0, 1 << 16),
       alg=st.sampled_from(["meshslice", "collective", "wang", "summa"]))
def test_every_dataflow_equals_the_dense_product(mesh, K, B, mi, ki, ni, seed, alg):
    R, C = mesh
    unit = K * B * R * C                      # divisible by every slicing the algorithms apply
    if alg == "wang":
        unit *= 2                             # the ring moves two half blocks per shard
    M, Kd, N = unit * mi, unit * ki, unit * ni
    g = torch.Generator().manual_seed(seed)
    X, W = torch.randn(M, Kd, generator=g, dtype=torch.float64), torch.randn(Kd, N, generator=g, dtype=torch.float64)
    m = EmuMesh(R, C)
    spmd = tp.SPMD(m, alg, blocksize=B)
    Y = X @ W
    y = m.unshard(spmd.OS(K)(m.shard(X), m.shard(W)))
    assert torch.allclose(y, Y, atol=1e-9, rtol=1e-9)
    dx = m.unshard(spmd.LS(K)(m.shard(Y), m.shard(W)))          # Y W^T
    assert torch.allclose(dx, Y @ W.t(), atol=1e-8, rtol=1e-9)
    dw = m.unshard(spmd.RS(K)(m.shard(X), m.shard(Y)))          # X^T Y
    assert torch.allclose(dw, X.t() @ Y, atol=1e-8, rtol=1e-9)


@settings(max_examples=50, deadline=None)
@given(K=st.integers(1, 8), B=st.integers(1, 16), reps=st.integers(1, 5))
def test_slices_partition_the_index_range(K, B, reps):
    length = K * B * reps
    seen = torch.cat([tp.slice_indices(length, K, B, i) for i in range(K)])
    assert sorted(seen.tolist()) == list(range(length))
    for i in range(K):
        idx = tp.slice_indices(length, K, B, i)
        assert len(idx) == length // K and all(((int(v) // B) % K) == i for v in idx)
    if K * B > 1:      # a length that K * B does not divide is refused
        with pytest.raises(ValueError):
            tp.slice_indices(length + 1, K, B, 0)


@settings(max_examples=60, deadline=None)
@given(tm=st.integers(1, 12), tn=st.integers(1, 12), sd=st.sampled_from([0, 1]), S=st.sampled_from([1, 2, 3, 4]),
       cyc=st.sampled_from([1, 2]), group=st.sampled_from([1, 3, 4, 8]), rot_frac=st.floats(0, 0.99))
def test_tile_map_is_a_permutation_for_any_schedule(tm, tn, sd, S, cyc, group, rot_frac):
    tiles_s = tm if sd == 0 else tn
    if tiles_s % (S * cyc):
        return
    nb = tiles_s // S
    d = dict(M=tm * 256, N=tn * 256, slice_dim=sd, n_slices=S, cyc=cyc, group=group, rot=int(rot_frac * nb))
    sched = fz.tile_schedule(d)
    assert sorted((a, b) for a, b, _ in sched) == [(i, j) for i in range(tm) for j in range(tn)]
    # slices are visited one after another, and a block of the sliced dimension belongs to one slice only
    order = [s for _, _, s in sched]
    assert order == sorted(order)
    owner = {}
    for a, b, s in sched:
        blk = a if sd == 0 else b
        assert owner.setdefault(blk, s) == s
        assert (blk // cyc) % S == s
