"""Python front end of the stand-alone network simulator (``csrc/netsim``).

Builds the simulator with the host C++ compiler, runs scenarios and host programs, and turns
simulated collective sweeps into the fabric constants that the cost model and the autotuner
consume — "which mesh shape and slice counts would the tuner pick on *that* fabric" without owning
the fabric.  The reference keeps its simulator and its autotuner apart (the constants of
Autotuner.py:12-19 were typed in by hand from measurements); this module closes the loop.

    python -m meshslice_b200.utils.netsim run --scenario imb --nodes 2 --bytes 1
    python -m meshslice_b200.utils.netsim fit --config b200_nvswitch.ini --rows 2 --cols 4 --out fabric_sim.json
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

SRC_DIR = Path(__file__).resolve().parent.parent / "csrc" / "netsim"
SOURCES = ("netsim.cc", "scenarios.cc", "host.cc", "mpi.cc", "apps.cc", "config.cc", "main.cc")
CONFIG_DIR = SRC_DIR / "configs"


class NetsimError(RuntimeError):
    pass


def _fingerprint() -> str:
    h = hashlib.sha1()
    for f in sorted(SRC_DIR.glob("*.cc")) + sorted(SRC_DIR.glob("*.h")):
        h.update(f.name.encode())
        h.update(f.read_bytes())
    return h.hexdigest()[:16]


def build(force: bool = False) -> Path:
    """Compiles the simulator once per source state and returns the binary's path."""
    cxx = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        raise NetsimError("no C++ compiler found (set CXX)")
    cache = Path(os.environ.get("MSB_NETSIM_CACHE", SRC_DIR / ".build"))
    try:
        cache.mkdir(parents=True, exist_ok=True)
        if not os.access(cache, os.W_OK):
            raise PermissionError(str(cache))
    except OSError:      # read-only installation: fall back to the system's scratch directory
        cache = Path(tempfile.gettempdir()) / "meshslice_b200_netsim"
        cache.mkdir(parents=True, exist_ok=True)
    exe = cache / f"netsim-{_fingerprint()}"
    if exe.exists() and not force:
        return exe
    cmd = [cxx, "-std=c++20", "-O2", "-Wno-psabi", "-o", str(exe) + ".tmp", *[str(SRC_DIR / s) for s in SOURCES]]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise NetsimError("netsim build failed:\n" + r.stderr[-4000:])
    os.replace(str(exe) + ".tmp", exe)
    return exe


def config_path(name_or_path: Optional[str]) -> Optional[str]:
    """A shipped system description by name (``sst_torus.ini`` ...) or any ini file by path."""
    if not name_or_path:
        return None
    p = Path(name_or_path)
    if p.exists():
        return str(p)
    q = CONFIG_DIR / name_or_path
    if q.exists():
        return str(q)
    raise NetsimError(f"no such system description: {name_or_path}")


def run(scenario: str, nodes: Optional[int] = None, nbytes: Optional[int] = None, topology: Optional[str] = None,
        repeat: Optional[int] = None, config: Optional[str] = None, settings: Optional[Dict[str, object]] = None,
        timeout: float = 600.0) -> dict:
    """Runs one scenario / host program and returns the simulator's JSON record.
    ``settings`` are ``{"section.key": value}`` overrides on top of ``config``."""
    cmd = [str(build())]
    cfg = config_path(config)
    if cfg:
        cmd += ["--config", cfg]
    cmd += ["--scenario", scenario]
    for flag, v in (("--nodes", nodes), ("--bytes", nbytes), ("--topology", topology), ("--repeat", repeat)):
        if v is not None:
            cmd += [flag, str(v)]
    for k, v in (settings or {}).items():
        cmd += ["--set", f"{k}={v}"]
    r = subprocess.run(cmd + ["--json"], capture_output=True, text=True, timeout=timeout)
    if r.returncode == 2:
        raise NetsimError(r.stderr.strip() or "netsim rejected its arguments")
    try:
        out = json.loads(r.stdout)
    except json.JSONDecodeError as e:
        raise NetsimError(f"unreadable simulator output: {r.stdout[-500:]} {r.stderr[-500:]}") from e
    if not out.get("ok"):
        raise NetsimError(f"scenario {scenario} failed: {out.get('error', 'unknown error')}")
    return out


def sweep(scenario: str, sizes: Iterable[int], value: str, **kw) -> List[Tuple[int, float]]:
    """(bytes, seconds) points of one scenario over message sizes; ``value`` names the field (in us)."""
    return [(int(s), run(scenario, nbytes=int(s), **kw)[value] * 1e-6) for s in sizes]


def _fit(points: Sequence[Tuple[int, float]]) -> Tuple[float, float]:
    """Intercept from the smallest sizes, slope (s/byte) by least squares on the upper half."""
    import numpy as np
    s = np.array([p[0] for p in points], dtype=float)
    t = np.array([p[1] for p in points], dtype=float)
    hi = s >= np.median(s)
    slope = float(np.polyfit(s[hi], t[hi], 1)[0])
    return float(t[:2].mean()), slope


def fit_fabric(rows: int, cols: int, config: Optional[str] = None, topology: str = "crossbar",
               sizes: Sequence[int] = (1 << 10, 1 << 12, 1 << 14, 1 << 16, 1 << 18, 1 << 20, 1 << 22),
               direct: Optional[bool] = None, flops_per_chip: float = 1.38e15) -> dict:
    """Fabric constants (the autotuner's ``FabricConstants`` dictionary) from simulated sweeps.

    Each mesh axis is simulated as its own group of ``n`` nodes on ``topology`` ("crossbar", or
    "torus" for a ring of ``n``): all-gather with one-sided transfers (direct stores to every peer
    on a switch, neighbour forwarding on a ring) and the send-receive ring shift.  A reduce-scatter
    moves the same bytes as an all-gather in the opposite direction and is given the same
    constants."""
    if direct is None:
        direct = topology.startswith("crossbar")
    lat, bws, base = {}, {}, {}
    ag_kind = "allgather-direct" if direct else "allgather-ring"
    per_axis = {}
    for axis, n in (("rows", rows), ("cols", cols)):
        if n < 2:
            continue
        topo = topology if topology.startswith("crossbar") else f"torus:{n}"
        ag = sweep(ag_kind, sizes, "collective_us", nodes=n, topology=topo, config=config)
        sr = sweep("sendrecv", sizes, "exchange_us", nodes=n, topology=topo, config=config)
        a_ag, b_ag = _fit(ag)
        a_sr, b_sr = _fit(sr)
        per_axis[axis] = dict(ag=(a_ag, (n - 1) / b_ag, n - 1), sr=(a_sr, 1.0 / b_sr, 1))
    if not per_axis:
        raise NetsimError("a 1 x 1 mesh has no fabric to fit")
    first = next(iter(per_axis.values()))
    ring = not topology.startswith("crossbar")
    for kind, key in (("allgather", "ag"), ("reducescatter", "ag"), ("sendrecv", "sr")):
        if ring:
            # a ring collective pays the per-step latency once per forwarding step: split the
            # small-message time of every axis by its step count
            lat[kind] = min(v[key][0] / v[key][2] for v in per_axis.values())
            base[kind] = max(0.0, min(v[key][0] - lat[kind] * v[key][2] for v in per_axis.values()))
        else:
            a0 = min(v[key][0] for v in per_axis.values())
            lat[kind] = min(a0 / 2, 5e-6)
            base[kind] = max(a0 - lat[kind], 0.0)
        bws[kind] = [per_axis.get("rows", first)[key][1], per_axis.get("cols", first)[key][1]]
    return dict(latencies=lat, bws=bws, base_overheads=base,
                fabric="switch" if topology.startswith("crossbar") else "ring",
                shared_port=topology.startswith("crossbar"), flops_per_chip=flops_per_chip,
                mesh=[rows, cols], source=f"netsim {topology} {config or 'defaults'}")


def main(argv=None):
    ap = argparse.ArgumentParser(description="network simulator front end")
    sub = ap.add_subparsers(dest="cmd", required=True)
    r = sub.add_parser("run", help="run one scenario and print its JSON record")
    r.add_argument("--scenario", default="msg")
    r.add_argument("--nodes", type=int)
    r.add_argument("--bytes", type=int, dest="nbytes")
    r.add_argument("--topology")
    r.add_argument("--repeat", type=int)
    r.add_argument("--config")
    r.add_argument("--set", action="append", default=[], metavar="section.key=value")
    f = sub.add_parser("fit", help="fit the autotuner's fabric constants from simulated sweeps")
    f.add_argument("--rows", type=int, default=2)
    f.add_argument("--cols", type=int, default=4)
    f.add_argument("--topology", default="crossbar")
    f.add_argument("--config")
    f.add_argument("--out", default="")
    a = ap.parse_args(argv)
    if a.cmd == "run":
        settings = dict(kv.split("=", 1) for kv in a.set)
        print(json.dumps(run(a.scenario, a.nodes, a.nbytes, a.topology, a.repeat, a.config, settings)))
    else:
        d = fit_fabric(a.rows, a.cols, a.config, a.topology)
        text = json.dumps(d, indent=1)
        if a.out:
            Path(a.out).write_text(text)
        print(text)
    return 0


if __name__ == "__main__":
    sys.exit(main())
