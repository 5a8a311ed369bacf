#!/usr/bin/env python
"""Fit the cost model of the fused GEMM + collective kernel to measured 2-D GeMM sweeps (runs on CPU).

    python bench/fit_fused_model.py sweep.log [more.json ...] [--fabric-json in.json] [--out out.json]

Input: what `bench/BenchGemm2D.py` prints or writes with `--json` (one record per global shape, mesh and
dataflow, with the fused kernel's time per slice count).  The seven constants of
`meshslice_b200.cost_model.FusedKernelConstants` are fitted by least squares on log(predicted / measured)
over all (shape, mesh, dataflow, slices) points; the result is printed with the per-point ratios and, with
`--out`, written as the `fused` section of a fabric JSON that `run_autotune.py --fabric-json` reads.
"""
import argparse
import json
import math
import os
import sys

import numpy as np
from scipy.optimize import least_squares

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from meshslice_b200 import cost_model as cm  # noqa: E402
from meshslice_b200.autotuner import B200_NVSWITCH, FabricConstants  # noqa: E402

NAMES = ["launch_overhead", "gather_bw_alone", "gather_bw_overlap", "push_bw", "slot_sum_bw", "tile_eff",
         "slice_overhead"]
LOWER = [1e-5, 1e11, 5e10, 5e10, 2e11, 0.5, 1e-8]
UPPER = [5e-4, 9e11, 9e11, 9e11, 7e12, 1.3, 1e-4]


def read_rows(paths):
    rows = []
    for p in paths:
        text = open(p).read()
        try:
            d = json.loads(text)
            rows += d if isinstance(d, list) else d.get("rows", [d])
            continue
        except json.JSONDecodeError:
            pass
        for line in text.splitlines():
            line = line.strip()
            if line.startswith("{") and '"dataflow"' in line:
                rows.append(json.loads(line))
    return [r for r in rows if "fused" in r]


def points(rows):
    pts = []
    for r in rows:
        for s, v in r["fused"].items():
            pts.append((tuple(r["mesh"]), r["dataflow"], r["M"], r["N"], r["K"], int(s), v["ms"] * 1e-3))
    return pts


def predict(fabric, consts, pt):
    shape, df, M, N, K, s, _ = pt
    mesh = fabric.mesh(shape)
    mesh.fused = consts
    fn = {"os": cm.Fused_OS, "ls": cm.Fused_LS, "rs": cm.Fused_RS}[df]
    return sum(fn(mesh, M, N, K, s))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("inputs", nargs="+")
    ap.add_argument("--fabric-json", default="")
    ap.add_argument("--out", default="")
    ap.add_argument("--peak-tflops", type=float, default=1380.6, help="rate of the matmul estimator at efficiency 1")
    args = ap.parse_args(argv)
    fabric_dict = json.load(open(args.fabric_json)) if args.fabric_json else dict(B200_NVSWITCH)
    fabric = FabricConstants.from_dict(fabric_dict)
    pts = points(read_rows(args.inputs))
    if not pts:
        raise SystemExit("no sweep records found")

    def consts_of(x):
        return cm.FusedKernelConstants(matmul_peak=args.peak_tflops * 1e12,
                                       **{n: float(math.exp(v)) for n, v in zip(NAMES, x)})

    def resid(x):
        c = consts_of(x)
        return [math.log(predict(fabric, c, p) / p[-1]) for p in pts]

    x0 = [math.log(max(getattr(cm.FusedKernelConstants(), n), lo)) for n, lo in zip(NAMES, LOWER)]
    fit = least_squares(resid, x0, bounds=(np.log(LOWER), np.log(UPPER)))
    c = consts_of(fit.x)
    ratios = np.exp(np.array(resid(fit.x)))
    print("fitted constants:")
    for n in NAMES:
        print(f"  {n} = {getattr(c, n):.4g}")
    print(f"{len(pts)} points: predicted / measured median {np.median(ratios):.3f}, "
          f"within 10 %: {int((np.abs(ratios - 1) <= 0.10).sum())}, within 20 %: {int((np.abs(ratios - 1) <= 0.20).sum())}, "
          f"min {ratios.min():.2f}, max {ratios.max():.2f}")
    print("| mesh | dataflow | M x K x N | slices | measured ms | predicted ms | ratio |")
    print("|---|---|---|---|---|---|---|")
    for p, r in zip(pts, ratios):
        shape, df, M, N, K, s, t = p
        print(f"| {shape[0]}x{shape[1]} | {df} | {M} x {K} x {N} | {s} | {t * 1e3:.3f} | {t * r * 1e3:.3f} | {r:.2f} |")
    # does the model rank the slice counts of a case the way the measurement does?
    cases, agree = {}, 0
    for p, r in zip(pts, ratios):
        cases.setdefault(p[:5], []).append((p[5], p[6], p[6] * r))
    multi = [v for v in cases.values() if len(v) > 1]
    for v in multi:
        best_meas = min(v, key=lambda e: e[1])
        best_pred = min(v, key=lambda e: e[2])
        agree += best_pred[1] <= 1.10 * best_meas[1]
    print(f"slice count picked by the model within 10 % of the best measured one: {agree} of {len(multi)} cases")
    if args.out:
        fabric_dict["fused"] = c.to_dict()
        with open(args.out, "w") as f:
            json.dump(fabric_dict, f, indent=1)
        print("wrote", args.out)
    return c


if __name__ == "__main__":
    main()
