"""Cost model formulas and autotuner decisions with fixed fabric constants."""
import json
import math

import pytest

from meshslice_b200 import autotuner as AT
from meshslice_b200 import cost_model as CM


def _mesh(shape, consts=AT.TPUV4, matmul=None):
    return AT.FabricConstants.from_dict(consts).mesh(shape, matmul=matmul)


class ConstMatmul(CM.MatmulEstimator):
    def __init__(self, flops):
        self.flops = flops

    def __call__(self, M, N, K, layout="nn"):
        return 2.0 * M * N * K / self.flops


def test_ring_allgather_matches_reference_formula():
    mesh = _mesh((4, 8))
    shape = (1024, 512)
    size = 1024 * 512 * 2
    t = CM.estimateAllgather(mesh, shape, 1)
    assert t == pytest.approx(13e-6 + 7 * size / 79.751e9 + 7 * 5e-6)
    t0 = CM.estimateReduceScatter(mesh, shape, 0)
    assert t0 == pytest.approx(26e-6 + 3 * size / 37.506e9 + 3 * 5e-6)
    assert CM.estimateAllgather(_mesh((1, 8)), shape, 0) == 0.0


def test_switch_fabric_has_no_hop_latency_and_shares_the_port():
    mesh = _mesh((2, 4), AT.B200_NVSWITCH)
    size = 4096 * 1024 * 2
    t = CM.estimateAllgather(mesh, (4096, 1024), 1)
    assert t == pytest.approx(6e-6 + 3e-6 + 3 * size / 700e9)
    assert mesh.combine(1.0, 2.0) == 3.0
    assert _mesh((2, 4)).combine(1.0, 2.0) == 2.0


def test_hierarchical_dimension_folds_submesh():
    m = CM.DeviceMesh(((2, 4), 4), 1e15, AT.TPUV4["bws"], AT.TPUV4["latencies"], AT.TPUV4["base_overheads"])
    assert m.shape == (8, 4) and m.meshdim == 0 and m.submesh == (2, 4)
    assert CM.estimateAllgather(m, (256, 256), 0) > 0


def test_broadcast_reduce_and_cannon_models_run():
    """These paths raise in the reference (unassigned bw, missing precision argument)."""
    mesh = _mesh((4, 4), matmul=ConstMatmul(2e14))
    for f in (CM.SUMMA_OS, CM.SUMMA_LS, CM.SUMMA_RS, CM.Cannon_OS, CM.Cannon_LS, CM.Cannon_RS,
              CM.GSPMD_OS, CM.GSPMD_LS, CM.GSPMD_RS, CM.MeshFlow_OS, CM.MeshFlow_LS, CM.MeshFlow_RS,
              CM.LogicalRing_ISplit, CM.LogicalRing_WSplit, CM.LogicalRing_OSplit):
        pro, steady = f(mesh, 8192, 8192, 8192, 4)
        assert pro >= 0 and steady > 0
    assert CM.tup2ms((0.001, 0.002))[2].startswith("3.0")


def test_meshslice_model_hides_communication_behind_compute():
    mesh = _mesh((2, 4), AT.B200_NVSWITCH, matmul=ConstMatmul(1.4e15))
    M, N, K = 65536, 12288, 4096
    sliced = sum(CM.MeshFlow_OS(mesh, M, N, K, 8))
    unsliced = sum(CM.GSPMD_OS(mesh, M, N, K))
    compute = 2.0 * M * N * K / 8 / 1.4e15
    assert compute < sliced < unsliced
    # more slices shrink the exposed prologue
    assert CM.MeshFlow_OS(mesh, M, N, K, 8)[0] < CM.MeshFlow_OS(mesh, M, N, K, 2)[0]


def test_dataflow_rule_keeps_largest_matrix_stationary():
    assert AT.FFLayerModel(65536, 4096, 12288).dataflow == "os"
    assert AT.FFLayerModel(65536, 16384, 4096).dataflow == "ls"
    assert AT.FFLayerModel(65536, 4096, 4096).dataflow == "ls"
    assert AT.FFLayerModel(512, 4096, 16384).dataflow == "rs"


def test_possible_k_respects_divisibility_on_both_axes():
    ks = AT.possibleK(65536, 12288, 49152, (4, 8), "os")     # kdim = 12288/8/8 = 192
    assert ks == [k for k in range(3, 25) if 192 % k == 0]
    for k in AT.possibleK(65536, 4096, 16384, (2, 4), "os", blocksize=64):
        assert (4096 // 4) % (k * 64) == 0 and (4096 // 2) % (k * 64) == 0
    assert AT.possibleK(16, 64, 64, (2, 4), "os") == [2]


def test_autotuner_gpt3_block_decisions_tpuv4_constants():
    g = AT.build_transformerBlock(32, 2048, 96, 128)
    shapes = [(4, 8), (8, 4), (2, 16), (16, 2)]
    t = AT.Autotuner(g, shapes, matmul=ConstMatmul(2.6e14), verbose=False)
    flows = [t.dataflows[n] for n, *_ in g.ff_layers()]
    assert flows == ["os", "ls", "os", "ls"]
    assert not any(t.transposition.values())
    assert t.bestshape in shapes
    best = t.emulatedFinetune(sweep=True)
    times = {s: t.emulateFFTime(s)[0] for s in shapes}
    assert times[best] == pytest.approx(min(times.values()))
    res = t.result()
    assert res["mesh"] == list(best) and len(res["layers"]) == 4 and all(l["ksplit"] for l in res["layers"])


def test_transpose_nodes_inserted_when_an_rs_layer_flips_orientation():
    g = AT.ComputeGraph()
    x = g.Input([1, 256, 1024])
    f = g.FeedForward(x, 1024)          # tokens (256) smaller than both feature dims -> 'rs'
    g.Add(x, f)
    t = AT.Autotuner(g, [(2, 4)], matmul=ConstMatmul(1e15), verbose=False)
    assert list(t.dataflows.values()) == ["rs"]
    kinds = [g.nodes[n]["op_type"] for n in g.nodenames]
    assert kinds == ["Input", "FeedForward", "Transpose", "Add"]
    add = g.nodes[g.nodenames[-1]]
    assert any(i.startswith("Transpose") for i in add["inputs"])


def test_fabric_json_roundtrip_and_cli(tmp_path):
    p = tmp_path / "fabric.json"
    json.dump(AT.B200_NVSWITCH, open(p, "w"))
    fc = AT.FabricConstants.load(p)
    assert fc.fabric == "switch" and fc.bws["allgather"] == (700e9, 700e9)
    out = tmp_path / "tuned.json"
    AT.main(["--nrows", "2", "--ncols", "4", "--batchsize", "32", "--nheads", "32", "--fabric-json", str(p),
             "--tuned-json", str(out), "--sweep"])
    tuned = json.load(open(out))
    assert tuned["mesh"] in ([1, 8], [2, 4], [4, 2], [8, 1])


# ---- model of the fused GEMM + collective kernel ----------------------------------------------
def _b200_mesh(shape, **consts):
    fab = AT.FabricConstants.from_dict(AT.B200_NVSWITCH)
    mesh = fab.mesh(shape)
    mesh.fused = CM.FusedKernelConstants(**consts)
    return mesh


def test_fused_model_on_one_gpu_is_the_tile_time_only():
    mesh = _b200_mesh((1, 1))
    for fn, layout in ((CM.Fused_OS, "nn"), (CM.Fused_LS, "nt"), (CM.Fused_RS, "tn")):
        pro, steady = fn(mesh, 8192, 8192, 4096, 4)
        assert pro == 0.0
        assert steady == pytest.approx(CM.AnalyticMatmul(1.3806e15, 1.0)(8192, 8192, 4096, layout) / 0.93)


def test_fused_model_slices_shrink_the_prologue_and_never_beat_the_tiles():
    mesh = _b200_mesh((2, 4))
    for fn in (CM.Fused_OS, CM.Fused_LS, CM.Fused_RS):
        p1, s1 = fn(mesh, 16384, 49152, 12288, 1)
        p4, s4 = fn(mesh, 16384, 49152, 12288, 4)
        assert p4 < p1
        assert p4 >= mesh.fused.launch_overhead
    # a product whose traffic dominates: the steady part is the transfer under tiles, not the tiles
    pro, steady = CM.Fused_OS(mesh, 16384, 4096, 4096, 4)
    tiles = CM.AnalyticMatmul(1.3806e15, 1.0)(16384 // 2, 4096 // 4, 4096, "nn") / 0.93
    assert steady >= tiles
    # exposed slot sums: with one slice the whole sum comes after the tiles, with eight an eighth of it
    (_, a), (_, b) = CM.Fused_LS(mesh, 16384, 16384, 4096, 1), CM.Fused_LS(mesh, 16384, 16384, 4096, 8)
    assert a > b


def test_fused_constants_are_recovered_from_a_synthetic_sweep(tmp_path):
    import importlib.util
    import os
    spec = importlib.util.spec_from_file_location(
        "fit_fused_model", os.path.join(os.path.dirname(__file__), "..", "bench", "fit_fused_model.py"))
    fit = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(fit)
    true = dict(launch_overhead=8e-5, gather_bw_alone=6e11, gather_bw_overlap=2.5e11, push_bw=4e11,
                slot_sum_bw=1.5e12, tile_eff=0.9, slice_overhead=5e-6)
    rows = []
    for shape in ((2, 4), (4, 2), (1, 8), (8, 1)):
        mesh = _b200_mesh(shape, **true)
        for (M, K, N) in ((16384, 4096, 16384), (16384, 16384, 4096), (16384, 12288, 49152), (16384, 49152, 12288)):
            for df, fn in (("os", CM.Fused_OS), ("ls", CM.Fused_LS), ("rs", CM.Fused_RS)):
                rows.append(dict(M=M, K=K, N=N, mesh=list(shape), dataflow=df,
                                 fused={str(s): {"ms": sum(fn(mesh, M, N, K, s)) * 1e3} for s in (1, 2, 4, 8)}))
    src = tmp_path / "sweep.log"
    src.write_text("noise line\n" + "\n".join(json.dumps(r) for r in rows) + "\n")
    out = tmp_path / "fabric.json"
    got = fit.main([str(src), "--out", str(out)])
    for k, v in true.items():
        assert getattr(got, k) == pytest.approx(v, rel=0.05), k
    # the autotuner picks the fused model up from the fabric file
    fab = AT.FabricConstants.load(str(out))
    assert fab.fused is not None and fab.mesh((2, 4)).fused.push_bw == pytest.approx(4e11, rel=0.05)
    layer = AT.FFLayerModel(65536, 4096, 16384, "os")
    t_fused = layer.emulate(fab.mesh((2, 4)), 4)
    fab.fused = None
    t_pipe = layer.emulate(fab.mesh((2, 4)), 4)
    assert t_fused > 0 and t_pipe > 0 and t_fused != t_pipe


def test_cli_meshes_restricts_the_candidates(tmp_path, capsys):
    out = tmp_path / "tuned.json"
    tuner = AT.main(["--nrows", "2", "--ncols", "4", "--batchsize", "16", "--nheads", "96", "--meshes", "4x2",
                     "--tuned-json", str(out)])
    assert tuple(tuner.bestshape) == (4, 2)
    d = json.load(open(out))
    assert d["mesh"] == [4, 2] and len(d["layers"]) == 4 and all(l["ksplit"] >= 1 for l in d["layers"])
    with pytest.raises(SystemExit):
        AT.main(["--nrows", "2", "--ncols", "4", "--meshes", "3x3"])
