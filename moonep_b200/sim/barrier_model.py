"""Host-side model of the device cross-rank barrier (csrc/device/prims.cuh):
every rank owns one epoch word per peer; arriving at barrier n stores n into slot [my rank]
of every peer, completion means every slot of my row has reached n. A wait that runs out of
budget returns a status record instead of blocking forever.  Used to test the failure paths
(a rank that never arrives, a dropped arrival) without touching a GPU.
"""

from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class BarrierStatus:
    ok: bool
    rank: int
    peer: int = -1
    observed: int = 0
    expected: int = 0


@dataclass
class EpochBarrierModel:
    R: int
    flags: list = field(default_factory=list)    # flags[r][p]: last epoch rank p announced to r
    epoch: list = field(default_factory=list)

    def __post_init__(self):
        self.flags = [[0] * self.R for _ in range(self.R)]
        self.epoch = [0] * self.R

    def arrive(self, rank: int, drop_to: set | None = None) -> int:
        """Rank announces its next epoch to every peer (except those in ``drop_to``)."""
        self.epoch[rank] += 1
        for p in range(self.R):
            if drop_to and p in drop_to:
                continue
            self.flags[p][rank] = self.epoch[rank]
        return self.epoch[rank]

    def wait(self, rank: int, polls: int = 1) -> BarrierStatus:
        """Bounded wait: succeeds iff every peer's slot reached this rank's epoch."""
        ep = self.epoch[rank]
        for _ in range(max(1, polls)):
            late = [p for p in range(self.R) if self.flags[rank][p] - ep < 0]
            if not late:
                return BarrierStatus(True, rank)
        p = late[0]
        return BarrierStatus(False, rank, p, self.flags[rank][p], ep)

    def reset(self):
        self.__post_init__()
