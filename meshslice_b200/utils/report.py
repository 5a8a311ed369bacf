"""Tables from run records.

``bench.py`` prints one JSON line per run and ``RunLogger`` writes one JSON object per event;
this module collects such lines from log files (anything that is not a JSON object is skipped)
and renders Markdown tables: a scaling table of benchmark runs and a per-step table of a
training log.  It replaces copying numbers by hand into result files.

    python -m meshslice_b200.utils.report bench_n1.log bench_n2.log bench_n8.log
    python -m meshslice_b200.utils.report --steps train.jsonl
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import Iterable, List


def read_records(paths: Iterable[str]) -> List[dict]:
    """Every JSON object found on its own line in the given files, in order."""
    out = []
    for p in paths:
        with open(p) as f:
            for line in f:
                line = line.strip()
                if not (line.startswith("{") and line.endswith("}")):
                    continue
                try:
                    rec = json.loads(line)
                except json.JSONDecodeError:
                    continue
                if isinstance(rec, dict):
                    rec.setdefault("_file", p)
                    out.append(rec)
    return out


def _fmt(v, nd=1):
    if v is None:
        return ""
    if isinstance(v, float):
        return f"{v:.{nd}f}"
    return str(v)


def scaling_table(records: List[dict]) -> str:
    """Benchmark lines (those with 'metric' and 'n_gpus') as a scaling table, one row per run,
    with the efficiency relative to the smallest GPU count of the same implementation."""
    runs = [r for r in records if "metric" in r and "n_gpus" in r and "value" in r]
    runs.sort(key=lambda r: (r.get("impl", ""), r["n_gpus"]))
    base = {}
    for r in runs:
        base.setdefault(r.get("impl", ""), r)
    head = "| impl | GPUs | parallelism | value | unit | per GPU | ms / step | efficiency | end to end | SM MHz | reasons |"
    rows = [head, "|" + "---|" * 11]
    for r in runs:
        b = base[r.get("impl", "")]
        per_gpu = r["value"] / r["n_gpus"]
        eff = per_gpu / (b["value"] / b["n_gpus"]) if b["value"] else None
        clocks = r.get("clocks") or {}
        rows.append("| " + " | ".join([
            r.get("impl", ""), str(r["n_gpus"]), (r.get("config") or {}).get("parallelism", ""), _fmt(float(r["value"])),
            r.get("unit", ""), _fmt(per_gpu), _fmt(r.get("ms_per_step")), _fmt(eff, 2),
            _fmt((r.get("e2e") or {}).get("value")), _fmt(clocks.get("sm_mhz"), 0), ", ".join(clocks.get("reasons", []))]) + " |")
    return "\n".join(rows)


def steps_table(records: List[dict]) -> str:
    """Events of kind 'step' from a RunLogger file."""
    steps = [r for r in records if r.get("kind") == "step"]
    keys = [k for k in ("step", "loss", "ms", "tokens_per_s", "tflops_per_gpu") if any(k in s for s in steps)]
    rows = ["| " + " | ".join(keys) + " |", "|" + "---|" * len(keys)]
    for s in steps:
        rows.append("| " + " | ".join(_fmt(s.get(k), 3 if k == "loss" else 1) for k in keys) + " |")
    return "\n".join(rows)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("files", nargs="+")
    ap.add_argument("--steps", action="store_true", help="per-step table of a training log instead of the scaling table")
    a = ap.parse_args(argv)
    recs = read_records(a.files)
    print(steps_table(recs) if a.steps else scaling_table(recs))
    return 0


if __name__ == "__main__":
    sys.exit(main())
