"""Host-side failure detection between engine steps.

Every rank of an SPMD job takes the same steps; a rank that is gone makes the next collective of the others wait
on a peer that will never arrive.  ``RankMonitor`` lets the others find out on the HOST, before they launch
anything that waits on that peer:

* a rank that leaves in an orderly way (between steps, with none of its kernels or collectives in flight) calls
  :meth:`leave`; the others see its ``left`` key at their next :meth:`check` and raise :class:`RankLeft`;
* a rank that dies without notice stops beating; :meth:`check` waits at most ``timeout`` seconds for every peer
  to have reached the previous step and raises :class:`RankTimeout` otherwise.

The state lives in the process group's key-value store (the TCP store every ``torch.distributed`` job already
has), so a check never touches a GPU stream or a device-side collective.  Device-side waits are bounded
separately (status words, see ``engine/runner.py``); the reference has no failure detection of its own.
"""
from __future__ import annotations

import time
from typing import Optional


class RankLeft(RuntimeError):
    """A peer announced that it left the job; no further collective with it may be launched."""


class RankTimeout(RuntimeError):
    """A peer did not reach the previous step within the time limit (crashed or hung on the host)."""


class RankMonitor:
    def __init__(self, store, rank: int, world_size: int, timeout: float = 30.0, prefix: str = "b200/health"):
        self.store, self.rank, self.world, self.timeout, self.prefix = store, rank, world_size, timeout, prefix
        self.step = 0
        self._left: set = set()
        self.store.set(self._k("hb", rank), "0")

    @classmethod
    def from_default_group(cls, timeout: float = 30.0) -> Optional["RankMonitor"]:
        import torch.distributed as dist
        if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
            return None
        from torch.distributed.distributed_c10d import _get_default_store
        return cls(_get_default_store(), dist.get_rank(), dist.get_world_size(), timeout)

    def _k(self, kind: str, rank: int) -> str:
        return f"{self.prefix}/{kind}/{rank}"

    def _get(self, key: str) -> Optional[bytes]:
        # ``check`` is the non-blocking probe of c10d stores (``get`` would wait for the key)
        return self.store.get(key) if self.store.check([key]) else None

    def beat(self) -> int:
        """Announce that this rank is about to enter its next step; pair with ``check(wait_for_step=step)`` for a
        host-side handshake in front of the step's collectives."""
        self.step += 1
        self.store.set(self._k("hb", self.rank), str(self.step))
        return self.step

    def leave(self, reason: str = "") -> None:
        """Orderly exit between steps: the caller has no kernel or collective in flight."""
        self.store.set(self._k("left", self.rank), reason or "left")

    def peers_left(self) -> dict:
        out = {}
        for r in range(self.world):
            if r != self.rank:
                v = self._get(self._k("left", r))
                if v is not None:
                    out[r] = v.decode() if isinstance(v, bytes) else str(v)
        return out

    def check(self, wait_for_step: Optional[int] = None) -> None:
        """Raise if a peer left, or - when ``wait_for_step`` is given - if a peer has not reached that step in time.
        Call before launching a step that contains collectives."""
        gone = self.peers_left()
        if gone:
            raise RankLeft(f"rank(s) {sorted(gone)} left the job ({gone}); rank {self.rank} stops before its next launch")
        if wait_for_step is None:
            return
        deadline = time.monotonic() + self.timeout
        pending = [r for r in range(self.world) if r != self.rank]
        while pending:
            still = []
            for r in pending:
                v = self._get(self._k("hb", r))
                if v is None or int(v) < wait_for_step:
                    still.append(r)
            gone = self.peers_left()
            if gone:
                raise RankLeft(f"rank(s) {sorted(gone)} left the job ({gone})")
            pending = still
            if not pending:
                return
            if time.monotonic() > deadline:
                raise RankTimeout(f"rank(s) {pending} did not reach step {wait_for_step} within {self.timeout:.1f} s")
            time.sleep(0.002)
