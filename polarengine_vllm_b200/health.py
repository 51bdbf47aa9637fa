"""Host-side failure detection for the sharded decoder: ranks learn that a peer has left BEFORE their next launch.

The device-side exchange (``pe_allreduce_add_rmsnorm``) waits for every peer's flag with a bounded wait, so a missing
peer costs a second and a status word rather than a hung GPU -- but the cheap way out is not to launch at all.
Every rank publishes a step counter and, when it leaves between steps (an exception, a shutdown), a farewell note in
the job's key-value store; :meth:`RankMonitor.check` is called before each step and raises :class:`PeerLeft` or
:class:`PeerStale` on the survivors, which can then drain, re-shard or stop without any kernel or collective in
flight.  The reference has no counterpart (it has no multi-rank code at all; vLLM owns the process group).
"""
from __future__ import annotations

import time
from typing import Dict, Optional


class PeerLeft(RuntimeError):
    """A peer rank announced that it is leaving (``rank``, ``reason``)."""

    def __init__(self, rank: int, reason: str):
        super().__init__(f"rank {rank} left the job: {reason}")
        self.rank, self.reason = rank, reason


class PeerStale(RuntimeError):
    """A peer's step counter has not advanced within the allowed time (``rank``, ``age_s``)."""

    def __init__(self, rank: int, age_s: float):
        super().__init__(f"rank {rank} has not reported a step for {age_s:.1f} s")
        self.rank, self.age_s = rank, age_s


class RankMonitor:
    """``store`` is any torch.distributed store (TCPStore, FileStore, the default store of an initialised process
    group).  All operations are non-blocking on the failure path: ``check`` only reads keys that exist."""

    def __init__(self, store, rank: int, world: int, prefix: str = "polar_b200", stale_after_s: Optional[float] = None):
        self.store, self.rank, self.world, self.prefix = store, rank, world, prefix
        self.stale_after_s = stale_after_s
        self._seen: Dict[int, tuple] = {}  # peer -> (last counter, time it changed)
        self.beat(0)

    def _key(self, kind: str, rank: int) -> str:
        return f"{self.prefix}/{kind}/{rank}"

    def beat(self, step: int) -> None:
        """Publish this rank's step counter (call once per step, after the step's device work was queued)."""
        self.store.set(self._key("step", self.rank), str(int(step)))

    def leave(self, reason: str = "shutdown") -> None:
        """Announce that this rank leaves; call between steps, with none of its kernels or collectives in flight."""
        self.store.set(self._key("left", self.rank), reason or "shutdown")

    def check(self) -> None:
        """Raise if a peer has left, or (with ``stale_after_s``) stopped reporting steps.  Call before a launch."""
        now = time.monotonic()
        for peer in range(self.world):
            if peer == self.rank:
                continue
            if self.store.check([self._key("left", peer)]):
                raise PeerLeft(peer, self.store.get(self._key("left", peer)).decode())
            if self.stale_after_s is not None and self.store.check([self._key("step", peer)]):
                counter = int(self.store.get(self._key("step", peer)).decode())
                last = self._seen.get(peer)
                if last is None or last[0] != counter:
                    self._seen[peer] = (counter, now)
                elif now - last[1] > self.stale_after_s:
                    raise PeerStale(peer, now - last[1])
