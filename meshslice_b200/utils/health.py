"""Host-side failure detection for a group of ranks.

The reference has none (a failing ``jax.distributed.initialize`` simply raises).  Here every rank
publishes a heartbeat (its step counter, or a departure notice) in the job's key-value store
between steps, and checks its peers' entries before launching the next step: a rank that left or
raised is reported as ``PeerLostError`` on every surviving rank *before* they enter a collective
or a fused kernel that would wait for it.  Device-side waits are bounded separately (the kernels
report a status code instead of spinning), so a lost peer can never hang a GPU.
"""
from __future__ import annotations

import time
from typing import Optional


class PeerLostError(RuntimeError):
    pass


class Heartbeat:
    def __init__(self, store, rank: int, world: int, prefix: str = "hb"):
        self.store, self.rank, self.world, self.prefix = store, rank, world, prefix

    def _key(self, r):
        return f"{self.prefix}/{r}"

    def _peek(self, key: str) -> str:
        """Value of ``key`` or "" when nobody has set it yet.  ``store.get`` blocks until the key
        exists (for the store's own timeout, minutes by default), which would stall every survivor
        behind a peer that died before its first beat; ``check`` asks without blocking first."""
        try:
            if hasattr(self.store, "check") and not self.store.check([key]):
                return ""
            return self.store.get(key).decode()
        except Exception:
            return "unreachable"      # the store's host process is gone

    def beat(self, step: int):
        self.store.set(self._key(self.rank), f"step:{step}")

    def leave(self, reason: str = "left"):
        """Publish a departure notice (call between steps, with nothing in flight)."""
        self.store.set(self._key(self.rank), f"gone:{reason}")

    def check(self, step: int, timeout_s: float = 5.0):
        """Raises PeerLostError if a peer announced its departure or has not reached ``step``
        within ``timeout_s``."""
        deadline = time.time() + timeout_s
        for r in range(self.world):
            if r == self.rank:
                continue
            while True:
                v = self._peek(self._key(r))
                if v.startswith("gone:"):
                    raise PeerLostError(f"rank {r} left the job ({v[5:]}) before step {step}")
                if v.startswith("step:") and int(v[5:]) >= step:
                    break
                if time.time() > deadline:
                    if v == "unreachable":
                        raise PeerLostError(f"the job's key-value store stopped answering before step {step}: "
                                            f"the rank that hosts it has left")
                    raise PeerLostError(f"rank {r} did not reach step {step} within {timeout_s}s (last: {v or 'nothing'})")
                time.sleep(0.02)


def guarded_step(hb: Heartbeat, step: int, fn, timeout_s: float = 5.0):
    """Heartbeat, check the peers, run ``fn``; on any exception publish a departure notice so
    that the other ranks stop cleanly instead of waiting."""
    hb.beat(step)
    hb.check(step, timeout_s)
    try:
        return fn()
    except Exception as e:
        hb.leave(f"{type(e).__name__}: {e}")
        raise


class RemoteKernelError(RuntimeError):
    """Another rank's kernel reported an error status."""


def agree_on_status(local_code: int, group=None, device=None) -> None:
    """Makes a kernel error of ANY rank an exception on EVERY rank of ``group``.

    Every rank contributes the status code its own kernels reported since the last check (0 when
    nothing went wrong); the codes are max-reduced together with the reporting rank, so all ranks
    learn which rank failed and with what, and stop before the next step instead of running into
    bounded waits one after another.  One small all-reduce: meant to be called once per step.
    ``device`` selects where the two-element tensor lives (CPU for Gloo groups, the current GPU
    for NCCL groups)."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        if local_code:
            raise RemoteKernelError(f"kernel status {local_code} on this rank")
        return
    rank = dist.get_rank(group)
    # code in the high part, rank in the low part: the maximum names the failing rank as well
    packed = torch.tensor([int(local_code) * 65536 + (rank if local_code else 0)], dtype=torch.int64,
                          device=device or "cpu")
    dist.all_reduce(packed, op=dist.ReduceOp.MAX, group=group)
    worst = int(packed.item())
    if worst:
        code, who = divmod(worst, 65536)
        raise RemoteKernelError(f"kernel status {code} reported by rank {who}" +
                                (" (this rank)" if who == rank and local_code == code else ""))
