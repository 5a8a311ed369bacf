"""In-tree build of the native extension ``meshslice_b200/_C*.so`` for sm_100a.

The CUDA sources are compiled with ``nvcc -gencode arch=compute_100a,code=sm_100a`` (this
cross-compiles on a machine without a GPU), the pybind11 bindings with the host compiler, and
everything is linked into one shared object next to the Python package so that it can be
imported without any JIT step.  ``python -m meshslice_b200.build`` rebuilds what is stale.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "csrc" / "build"

CU_SOURCES = [
    "gemm/sm100_gemm.cu",
    "gemm/sm100_gemm2.cu",
    "ops/ops.cu",
    "ops/attention.cu",
    "ops/attention_noalloc.cu",
    "comm/p2p.cu",
]
CPP_SOURCES = ["bindings.cpp"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; the native extension cannot be built")
    return cand


def ext_path() -> Path:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return PKG / f"_C{suffix}"


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def _headers():
    """Headers the CUDA / binding sources may include (the stand-alone simulator has its own build)."""
    hs = list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.cuh"))
    return [str(p) for p in hs if "netsim" not in p.parts]


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build step failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
    return r.stdout + r.stderr


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile every CUDA/C++ source that is newer than its object and relink if needed."""
    import pybind11

    OBJ.mkdir(parents=True, exist_ok=True)
    nvcc = _nvcc()
    headers = _headers()
    py_inc = sysconfig.get_paths()["include"]
    jobs = []
    objs = []
    for src in CU_SOURCES:
        s = CSRC / src
        if not s.exists():
            continue
        o = OBJ / (src.replace("/", "_") + ".o")
        objs.append(o)
        if force or _stale(o, [s] + headers):
            jobs.append([nvcc, *NVCC_FLAGS, "-Xptxas", "-v", "-I", str(CSRC), "-c", str(s), "-o", str(o)])
    for src in CPP_SOURCES:
        s = CSRC / src
        o = OBJ / (src.replace("/", "_") + ".o")
        objs.append(o)
        if force or _stale(o, [s] + headers):
            jobs.append([nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-I", pybind11.get_include(), "-I", py_inc,
                         "-x", "cu", "-c", str(s), "-o", str(o)])
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for out in ex.map(_run, jobs):
                if verbose:
                    print(out)
    target = ext_path()
    if force or jobs or _stale(target, objs):
        _run([nvcc, "-shared", "-o", str(target), *map(str, objs), "-cudart", "static"])
    return target


if __name__ == "__main__":
    p = build(verbose="-v" in sys.argv, force="--force" in sys.argv)
    print(p)
