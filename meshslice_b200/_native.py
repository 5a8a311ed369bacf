"""Loader of the in-tree native extension and the per-process kernel status word.

The extension is a plain pybind11 module (``meshslice_b200/_C*.so``) built by
``meshslice_b200.build``.  On a machine with a GPU a missing extension is an error: no op of
this package silently falls back to another implementation of a CUDA path.
"""
from __future__ import annotations

import importlib.util
import threading

_lock = threading.Lock()
_mod = None
_status = None

STATUS_NAMES = {
    0: "ok", 1: "timeout: producer waiting for a free stage", 2: "timeout: MMA waiting for TMA data",
    3: "timeout: MMA waiting for the epilogue", 4: "timeout: epilogue waiting for the accumulator",
    5: "timeout: waiting for a gathered chunk", 6: "timeout: bulk copy of the communication warp",
    7: "timeout: entry barrier with peers", 8: "timeout: exit barrier with peers",
    9: "timeout: reduce phase waiting for peers' partial tiles", 10: "timeout: waiting for the local go flag",
}


class KernelStatusError(RuntimeError):
    """A kernel of this package gave up on a bounded wait and reported an error code."""


def load():
    """Import (building if necessary and possible) and return the native module."""
    global _mod
    if _mod is not None:
        return _mod
    with _lock:
        if _mod is not None:
            return _mod
        from .build import ext_path
        path = ext_path()
        if not path.exists():
            from .build import build
            build()
        spec = importlib.util.spec_from_file_location("meshslice_b200._C", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _mod = mod
    return _mod


def available() -> bool:
    try:
        load()
        return True
    except Exception:
        return False


def stream_ptr() -> int:
    import torch
    return torch.cuda.current_stream().cuda_stream


class _Status:
    def __init__(self):
        C = load()
        self.host, self.dev = C.status_alloc()

    def read(self):
        return load().status_read(self.host)

    def clear(self):
        load().status_clear(self.host)


def status() -> _Status:
    """Host-mapped status word that every kernel launch of this process reports into."""
    global _status
    if _status is None:
        _status = _Status()
    return _status


def check_status(sync: bool = True) -> None:
    """Raise KernelStatusError if any kernel since the last check reported a timeout."""
    import torch
    if sync:
        torch.cuda.synchronize()
    st = status()
    code, blk, d0, d1 = st.read()
    if code != 0:
        st.clear()
        raise KernelStatusError(
            f"kernel status {code} ({STATUS_NAMES.get(code, '?')}), block {blk}, detail {d0}, {d1}")
