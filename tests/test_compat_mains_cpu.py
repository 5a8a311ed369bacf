"""The reference's scripts double as self-tests (`python TensorParallel.py wang` and so on); the
modules of the same names under meshslice_b200.compat keep that behaviour on emulated CPU meshes."""
import pytest

from meshslice_b200.compat import ShardedLayers, TensorParallel, TensorParallel1D


@pytest.mark.parametrize("alg", ["meshflow", "wang", "cannon", "summa"])
def test_2d_algorithm_self_test_prints_three_trues(alg, capsys):
    assert TensorParallel.main([alg]) == 0
    assert capsys.readouterr().out.split() == ["True"] * 3


def test_1d_self_test(capsys):
    assert TensorParallel1D.main([]) == 0
    assert capsys.readouterr().out.split() == ["True"] * 3


def test_block_benchmark_runs_on_an_emulated_mesh(capsys):
    assert ShardedLayers.main(["meshflow", "--iters", "1"]) == 0
    out = capsys.readouterr().out
    assert "forward" in out and "mesh 2x2" in out


def test_notebook_cells_execute():
    """The CPU walkthrough notebook stays runnable: its code cells are executed in order."""
    import json
    import os
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "notebooks", "MeshSliceCPU.ipynb")
    nb = json.load(open(path))
    ns = {}
    ran = 0
    for cell in nb["cells"]:
        if cell["cell_type"] == "code":
            exec(compile("".join(cell["source"]), f"<cell {ran}>", "exec"), ns)
            ran += 1
    assert ran >= 4 and all(ns["agree"].values()) and all(ns["checks"].values())
