"""Host-side liveness check of the ranks of an EP group.

Every collective kernel of this package waits on its peers, and although those waits are
bounded and report a status instead of hanging, a step that is launched while a peer is
already gone still burns its whole wait budget on the GPU.  ``PeerMonitor`` lets a training
loop notice a missing rank on the host, between steps, before it launches anything that would
wait for that rank: each rank publishes the number of the step it is about to run in a
key-value store (the process group's own store, or any ``torch.distributed.Store``) and then
checks that every peer has published the same step.  A rank that leaves on purpose says so;
a rank that died simply stops publishing and is reported after the timeout.

The reference has no counterpart (its barriers time out after ~100 s and trap the context,
moonep/_common.py:332-341).

    mon = PeerMonitor(store, rank, world)
    for step in range(n):
        mon.enter_step(step, timeout_s=5.0)     # raises PeerLost([...]) instead of launching
        train_step()
    mon.leave()
"""

from __future__ import annotations

import time


class PeerLost(RuntimeError):
    """Raised on the host when one or more ranks did not reach the step, or left."""

    def __init__(self, ranks, step, reason):
        self.ranks, self.step, self.reason = list(ranks), step, reason
        super().__init__(f"rank(s) {self.ranks} {reason} (step {step})")


_LEFT = b"left"


class PeerMonitor:
    def __init__(self, store, rank: int, world: int, prefix: str = "moonep/step"):
        self.store, self.rank, self.world, self.prefix = store, rank, world, prefix
        self._last_seen = {r: -1 for r in range(world)}

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self, step: int) -> None:
        """Publish that this rank is about to run ``step``."""
        self.store.set(self._key(self.rank), str(int(step)))

    def leave(self) -> None:
        """Publish that this rank stops taking part (call between steps, nothing in flight)."""
        self.store.set(self._key(self.rank), _LEFT)

    def _read(self, r: int):
        """Last published value of rank ``r``: an int step, ``"left"`` or None (nothing yet)."""
        key = self._key(r)
        try:
            if not self.store.check([key]):
                return None
            v = self.store.get(key)
        except Exception:            # the store's host is gone: that rank (and the store) is lost
            return "store"
        if v == _LEFT:
            return "left"
        try:
            return int(v)
        except ValueError:
            return None

    def missing(self, step: int) -> tuple[list[int], list[int]]:
        """``(behind, left)``: peers that have not published ``step`` yet, and peers that left."""
        behind, left = [], []
        for r in range(self.world):
            if r == self.rank:
                continue
            v = self._read(r)
            if v in ("left", "store"):
                left.append(r)
            elif v is None or v < step:
                behind.append(r)
            else:
                self._last_seen[r] = v
        return behind, left

    def enter_step(self, step: int, timeout_s: float = 5.0, poll_s: float = 0.01) -> None:
        """Publish ``step`` and return once every peer has published it too.  Raises
        ``PeerLost`` as soon as a peer has left, or after ``timeout_s`` for peers that never
        arrive.  Nothing is launched by this call, so the GPU is never left waiting."""
        try:
            self.beat(step)
        except Exception as exc:
            raise PeerLost([0], step, f"hosting the store is unreachable ({type(exc).__name__})") from exc
        deadline = time.monotonic() + timeout_s
        while True:
            behind, left = self.missing(step)
            if left:
                raise PeerLost(left, step, "left the group")
            if not behind:
                return
            if time.monotonic() >= deadline:
                raise PeerLost(behind, step, f"did not reach the step within {timeout_s:g} s")
            time.sleep(poll_s)
