"""Host restatement of the flagged dispatch's bookkeeping (csrc/device/dispatch_flagged.cu):
which rows go on the wire, in which order, and what the per-slot source table holds afterwards.

Of a token's slots on one destination rank, the one with the lowest slot offset names the unit of
work in the send list.  On a PEER rank only that slot receives the row and the token's other slots
there are duplicates whose ``rowsrc`` names it; on the sender's OWN rank every slot receives the row
directly (``rowsrc`` = the slot itself), since a local store costs no link bandwidth.  The send
list is ordered by bucket ``(slot // tile) * R + (d - rank) mod R``; the order inside a bucket is
unspecified (the device fills buckets with atomics), so it is compared bucket by bucket.
"""

from __future__ import annotations

import numpy as np

from .planner import ClusterPlan

FLAG_ROWS = 128


def wire_entries(cp: ClusterPlan, rank: int):
    """Entries ``s*K + k`` of ``rank`` whose row is sent, and the bucket of each (tile = FLAG_ROWS)."""
    raw = cp.dst_raw[rank].reshape(cp.S, cp.K).astype(np.int64)
    dest, loff = raw // cp.NvS, raw % cp.NvS
    out, buckets = [], []
    for s in range(cp.S):
        for k in range(cp.K):
            same = dest[s] == dest[s, k]
            if loff[s, k] == loff[s][same].min():
                out.append(s * cp.K + k)
                buckets.append((loff[s, k] // FLAG_ROWS) * cp.R + (dest[s, k] - rank) % cp.R)
    return np.asarray(out), np.asarray(buckets)


def rowsrc_tables(cp: ClusterPlan):
    """``rowsrc[d][slot]``: the slot whose payload a slot receives (itself for a row stored by the
    sender, the stored slot for a duplicate, -1 for a padding row); slots that no dispatch touches
    hold ``-2`` here."""
    tables = [np.full(cp.NvS, -2, dtype=np.int64) for _ in range(cp.R)]
    for d in range(cp.R):
        for g in range(cp.cu_seqlens.shape[1]):
            p0, n = (int(x) for x in cp.zero_fill_ranges[d, g])
            tables[d][p0:p0 + n] = -1
    for r in range(cp.R):
        raw = cp.dst_raw[r].reshape(cp.S, cp.K).astype(np.int64)
        dest, loff = raw // cp.NvS, raw % cp.NvS
        for s in range(cp.S):
            for k in range(cp.K):
                same = dest[s] == dest[s, k]
                d = int(dest[s, k])
                tables[d][int(loff[s, k])] = int(loff[s, k]) if d == r else int(loff[s][same].min())
    return tables
