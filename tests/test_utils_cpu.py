"""Run logging, report tables and trace helpers (no GPU)."""
import json

import torch

from meshslice_b200.utils import report
from meshslice_b200.utils.logging import RunLogger, read_jsonl
from meshslice_b200.utils.timing import annotate, trace


def test_run_logger_writes_one_json_object_per_event(tmp_path, capsys):
    path = tmp_path / "run.jsonl"
    log = RunLogger(str(path), rank=0)
    log.log("config", mesh="2x4", layers=4)
    for s in range(3):
        log.log("step", step=s + 1, loss=10.0 - s, ms=100.0 + s, tokens_per_s=1e5, tflops_per_gpu=700.0)
    log.close()
    recs = read_jsonl(str(path))
    assert [r["kind"] for r in recs] == ["config", "step", "step", "step"] and recs[3]["loss"] == 8.0
    assert "step:" in capsys.readouterr().err
    silent = RunLogger(str(tmp_path / "other.jsonl"), rank=3)      # only rank 0 writes
    silent.log("step", step=1)
    assert not (tmp_path / "other.jsonl").exists()
    table = report.steps_table(report.read_records([str(path)]))
    assert table.count("\n") == 4 and "| 3 | 8.000 | 102.0 |" in table


def test_scaling_table_from_benchmark_lines(tmp_path):
    lines = []
    for n, v in ((1, 1000.0), (2, 1800.0), (8, 5600.0)):
        lines.append(json.dumps({"metric": "m", "value": v, "unit": "TFLOP/s", "n_gpus": n, "ms_per_step": 2700.0 / (v / 1000),
                                 "impl": "meshslice_b200", "config": {"parallelism": f"mesh {n}"},
                                 "clocks": {"sm_mhz": 1500.0, "reasons": ["sw_power_cap"]}, "e2e": {"value": v - 1}}))
    f = tmp_path / "bench.log"
    f.write_text("NCCL version 2.28\nnot json {\n" + "\n".join(lines) + "\n{broken json}\n")
    recs = report.read_records([str(f)])
    assert len(recs) == 3
    table = report.scaling_table(recs)
    rows = table.splitlines()
    assert len(rows) == 5 and "| 0.70 |" in rows[4] and "| 0.90 |" in rows[3] and "sw_power_cap" in rows[2]
    assert report.main([str(f)]) == 0


def test_annotate_and_trace_work_without_a_gpu(tmp_path):
    with annotate("forward"):
        x = torch.ones(8) * 2
    assert x.sum().item() == 16
    with trace(None) as prof:
        assert prof is None
    out = tmp_path / "trace.json"
    with trace(str(out)):
        torch.ones(64, 64) @ torch.ones(64, 64)
    data = json.loads(out.read_text())
    assert "traceEvents" in data and len(data["traceEvents"]) > 0


def test_p2p_copy_jobs_are_checked_before_launch():
    import pytest
    from meshslice_b200.parallel.collectives import validate_copy_jobs, validate_reduce
    validate_copy_jobs([(4096, 8192, 4, 64, 64, 128)])
    for bad in [(4096, 8192, 4, 60, 64, 64),      # row of 30 bf16: the tail would be dropped
                (4096, 8200, 4, 64, 64, 64),      # destination not 16-byte aligned
                (4100, 8192, 4, 64, 64, 64),
                (4096, 8192, 4, 64, 72, 64),
                (4096, 8192, 4, 64, 64, 32),      # pitch smaller than the row
                (4096, 8192, 0, 64, 64, 64)]:
        with pytest.raises(ValueError):
            validate_copy_jobs([bad])
    validate_reduce([4096, 8192], 64, 16384, 32, 8, 32)
    with pytest.raises(ValueError):
        validate_reduce([4096, 8192], 64, 16384, 30, 8, 30)
    with pytest.raises(ValueError):
        validate_reduce([4096, 8194], 64, 16384, 32, 8, 32)


def test_logical_mesh_of_the_transformer_bench_maps_to_a_physical_one():
    import importlib.util
    import os
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench", "BenchTransformer.py")
    spec = importlib.util.spec_from_file_location("bench_transformer", path)
    bt = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bt)
    assert bt.physical_mesh(2, 4, 8) == (2, 4)
    assert bt.physical_mesh(4, 4, 8) == (2, 4)          # most square split that divides 4 x 4
    assert bt.physical_mesh(4, 4, 4) == (2, 2)
    assert bt.physical_mesh(8, 16, 8, "2x4") == (2, 4)
    assert bt.physical_mesh(4, 4, 1) == (1, 1)
    import pytest
    with pytest.raises(SystemExit):
        bt.physical_mesh(3, 3, 8)
    with pytest.raises(SystemExit):
        bt.physical_mesh(4, 4, 8, "8x1")


def test_fused_timeline_summary_and_chrome_export(tmp_path):
    """A synthetic launch: the gather runs from 0 to 100 us, tiles complete from 40 to 200 us, the slot sums of
    slice 0 run under the tiles and those of slice 1 after the last tile."""
    import json
    from meshslice_b200.utils.timing import fused_timeline_summary, fused_timeline_to_chrome
    ev = []
    for c in range(5):
        ev.append(dict(t_ns=c * 25_000, cta=c % 2, kind="chunk_sent", arg=c))
    for t in range(9):
        ev.append(dict(t_ns=40_000 + t * 20_000, cta=t % 2, kind="tile_computed", arg=t))
    ev += [dict(t_ns=120_000, cta=0, kind="sum_begin", arg=0), dict(t_ns=160_000, cta=0, kind="sum_end", arg=0),
           dict(t_ns=200_000, cta=0, kind="sum_begin", arg=1), dict(t_ns=240_000, cta=0, kind="sum_end", arg=1)]
    s = fused_timeline_summary(ev)
    assert s["tile_computed"]["count"] == 9 and s["chunk_sent"]["last_ns"] == 100_000
    assert s["overlap_chunks"] == 0.6          # 40..100 us of the 100 us gather lie after the first tile
    assert s["overlap_sums"] == 0.5            # slice 0 hidden, slice 1 exposed
    path = tmp_path / "timeline.json"
    fused_timeline_to_chrome(ev, str(path))
    recs = json.load(open(path))["traceEvents"]
    assert sum(r["ph"] == "X" for r in recs) == 2 and sum(r["ph"] == "i" for r in recs) == 14
