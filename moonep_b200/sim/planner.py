"""CPU oracle for the redundant-expert planner, all R ranks in one process.

It restates the planning semantics of the reference
(tests/planning_reference.py:25-311, moonep/planning.py:584-1098) without
``torch.distributed``: the caller passes every rank's top-k table and gets every
rank's plan back.  The device planner must reproduce these arrays exactly
(``dup_*`` as sets).  Heavy steps are numpy-vectorised so S=4096, R=8 runs in well
under a second.

Algorithm (identical on every rank because it only depends on the all-gathered
per-rank expert histograms):

1. ``count[e] = sum_r tpe[r, e]``; ``group[h] = sum`` over the ``epn`` experts homed
   on rank ``h``; ``balance = group - S*K``.
2. Receiver selection: repeatedly take the most loaded group ``h`` (lowest index on
   ties) and the emptiest rank ``u`` (lowest index on ties); stop when
   ``balance[h] <= 0``; ``u`` is filled to exactly ``S*K`` from ``h`` alone
   (``quota[h, u] = -balance[u]``).  Every receiver therefore has one remote home
   group and at most ``epn`` remote experts.
3. Expert split per home group: repeatedly give the receiver with the largest open
   quota tokens of the local expert with the most remaining tokens.
4. Layout per destination: local experts first (VM groups ``0..epn-1``), then the
   received experts in ascending global id (groups ``epn..2epn-1``); each non-empty
   group is padded to ``token_padding`` rows.
5. Destination of an entry: its index among all entries of the same expert
   (source-rank-major, then flat index) is looked up in the per-expert prefix over
   destination ranks.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np


@dataclass
class ClusterPlan:
    """Plans of all ranks plus the shared tables."""
    R: int
    E: int
    S: int
    K: int
    NvS: int
    token_padding: int
    tpe: np.ndarray               # [R, E]
    alloc: np.ndarray             # [E, R] tokens of expert e placed on rank d
    recv_from: np.ndarray         # [R] home group feeding rank d, or -1
    experts_to_copy: np.ndarray   # [R, epn]
    cu_seqlens: np.ndarray        # [R, 2epn]
    zero_fill_ranges: np.ndarray  # [R, 2epn, 2]
    remote_stats: np.ndarray      # [R, 2]
    expert_off: np.ndarray        # [R, E]
    dst_raw: np.ndarray           # [R, N] always >= 0
    dst: np.ndarray               # [R, N] duplicates encoded as -raw-1
    dup_tables: list              # per destination rank: {primary_loff: (dup loffs in k order)}


def solve_allocation(count: np.ndarray, R: int, cap: int):
    """Steps 1-3. Returns ``alloc[E, R]`` and ``recv_from[R]``, ``recv_amt[R]``."""
    E = count.shape[0]
    epn = E // R
    count = count.astype(np.int64)
    group = count.reshape(R, epn).sum(axis=1)
    assert int(group.sum()) == R * cap, "every rank must contribute exactly S*K entries"
    balance = group - cap
    recv_from = np.full(R, -1, dtype=np.int64)
    recv_amt = np.zeros(R, dtype=np.int64)
    for _ in range(R):
        h = int(np.argmax(balance))
        u = int(np.argmin(balance))
        if balance[h] <= 0:
            break
        move = -int(balance[u])
        assert recv_from[u] < 0
        recv_from[u] = h
        recv_amt[u] = move
        balance[h] -= move
        balance[u] = 0
    else:
        assert balance.max() <= 0, "receiver selection did not terminate"

    alloc = np.zeros((E, R), dtype=np.int64)
    alloc[np.arange(E), np.arange(E) // epn] = count
    for h in range(R):
        quotas = np.where(recv_from == h, recv_amt, 0)
        if quotas.max() <= 0:
            continue
        remaining = count[h * epn:(h + 1) * epn].copy()
        while True:
            d = int(np.argmax(quotas))
            if quotas[d] <= 0:
                break
            le = int(np.argmax(remaining))
            take = int(min(remaining[le], quotas[d]))
            assert take > 0, "quota exceeds the home group's tokens"
            e = h * epn + le
            alloc[e, d] += take
            alloc[e, h] -= take
            remaining[le] -= take
            quotas[d] -= take
    assert (alloc.sum(axis=1) == count).all()
    assert (alloc.sum(axis=0) <= cap).all()
    return alloc, recv_from, recv_amt


def layout_tables(alloc: np.ndarray, R: int, token_padding: int, NvS: int):
    """Step 4 for every destination rank."""
    E = alloc.shape[0]
    epn = E // R
    experts_to_copy = np.full((R, epn), -1, dtype=np.int64)
    cu = np.zeros((R, 2 * epn), dtype=np.int64)
    zfr = np.zeros((R, 2 * epn, 2), dtype=np.int64)
    stats = np.zeros((R, 2), dtype=np.int64)
    expert_off = np.zeros((R, E), dtype=np.int64)
    for d in range(R):
        lo, hi = d * epn, (d + 1) * epn
        col = alloc[:, d]
        remote = [int(e) for e in np.nonzero(col > 0)[0] if not (lo <= e < hi)]
        assert len(remote) <= epn, f"rank {d}: {len(remote)} remote experts exceed epn={epn}"
        stats[d, 0] = len(remote)
        for b, e in enumerate(remote):
            experts_to_copy[d, b] = e
            stats[e // epn, 1] += 1
        start = 0
        for g in range(2 * epn):
            e = lo + g if g < epn else int(experts_to_copy[d, g - epn])
            cnt = int(col[e]) if e >= 0 else 0
            padded = (cnt + token_padding - 1) // token_padding * token_padding if cnt > 0 else 0
            if cnt > 0:
                expert_off[d, e] = start
                if padded > cnt:
                    zfr[d, g] = (start + cnt, padded - cnt)
            start += padded
            cu[d, g] = start
        assert start <= NvS, "padded layout exceeds NvS"
    return experts_to_copy, cu, zfr, stats, expert_off


def plan_cluster(topk_all: np.ndarray, E: int, token_padding: int = 128, NvS: int | None = None) -> ClusterPlan:
    """Full plan for all ranks. ``topk_all`` is ``[R, S, K]`` integer expert ids."""
    topk_all = np.asarray(topk_all).astype(np.int64)
    R, S, K = topk_all.shape
    epn = E // R
    N = S * K
    if NvS is None:
        NvS = (N + (token_padding - 1) * 2 * epn + token_padding - 1) // token_padding * token_padding
    flat = topk_all.reshape(R, N)
    tpe = np.stack([np.bincount(flat[r], minlength=E) for r in range(R)]).astype(np.int64)
    count = tpe.sum(axis=0)
    alloc, recv_from, _ = solve_allocation(count, R, N)
    etc, cu, zfr, stats, expert_off = layout_tables(alloc, R, token_padding, NvS)

    alloc_cum = alloc.cumsum(axis=1)                      # [E, R]
    tpe_excl = np.concatenate([np.zeros((1, E), np.int64), tpe.cumsum(axis=0)[:-1]])  # [R, E]
    dst_raw = np.zeros((R, N), dtype=np.int64)
    for r in range(R):
        f = flat[r]
        order = np.argsort(f, kind="stable")
        pos = np.empty(N, dtype=np.int64)
        pos[order] = np.arange(N)
        expoff = np.concatenate([[0], np.cumsum(tpe[r])[:-1]])
        g = tpe_excl[r, f] + (pos - expoff[f])
        dest = (alloc_cum[f] <= g[:, None]).sum(axis=1)
        assert (dest < R).all()
        prev = np.where(dest > 0, alloc_cum[f, np.maximum(dest - 1, 0)], 0)
        dst_raw[r] = dest * NvS + expert_off[dest, f] + (g - prev)

    # duplicates: a later k of the same token going to an already used rank
    dest3 = (dst_raw // NvS).reshape(R, S, K)
    dup = np.zeros((R, S, K), dtype=bool)
    for k in range(1, K):
        dup[:, :, k] = (dest3[:, :, :k] == dest3[:, :, k:k + 1]).any(axis=2)
    dupf = dup.reshape(R, N)
    dst = np.where(dupf, -dst_raw - 1, dst_raw)

    dup_tables = [dict() for _ in range(R)]
    loff3 = (dst_raw % NvS).reshape(R, S, K)
    rr, ss, kk = np.nonzero(dup)
    for r, s, k in zip(rr.tolist(), ss.tolist(), kk.tolist()):
        d = int(dest3[r, s, k])
        kp = int(np.argmax(dest3[r, s] == d))
        p = int(loff3[r, s, kp])
        dup_tables[d].setdefault(p, []).append(int(loff3[r, s, k]))
    dup_tables = [{p: tuple(v) for p, v in t.items()} for t in dup_tables]

    return ClusterPlan(R, E, S, K, NvS, token_padding, tpe, alloc, recv_from, etc, cu, zfr, stats,
                       expert_off, dst_raw, dst, dup_tables)


def dup_table_from_arrays(dup_groups, dup_loffs, dup_counts) -> dict:
    """Decode device ``dup_*`` tensors into ``{primary: sorted tuple}`` (set semantics)."""
    g = np.asarray(dup_groups)
    lo = np.asarray(dup_loffs)
    ng = int(dup_counts[0])
    out = {}
    for j in range(ng):
        p, st, n = (int(x) for x in g[j])
        assert p not in out, f"primary row {p} listed twice"
        out[p] = tuple(sorted(int(x) for x in lo[st:st + n]))
    return out


def check_invariants(cp: ClusterPlan) -> None:
    """Structural guarantees a user may rely on (SxK real rows per rank etc.)."""
    R, E, N, NvS, pad = cp.R, cp.E, cp.S * cp.K, cp.NvS, cp.token_padding
    epn = E // R
    assert (cp.alloc.sum(axis=0) == N).all(), "every rank must receive exactly S*K rows"
    assert (cp.alloc.sum(axis=1) == cp.tpe.sum(axis=0)).all()
    for d in range(R):
        cu = cp.cu_seqlens[d]
        assert (np.diff(np.concatenate([[0], cu])) >= 0).all() and cu[-1] <= NvS
        assert (cu % pad == 0).all()
        remote = cp.experts_to_copy[d][cp.experts_to_copy[d] >= 0]
        assert len(set((remote // epn).tolist())) <= 1, "more than one remote home group"
        assert (np.diff(remote) > 0).all()
        # every slot is hit exactly once
        hits = np.zeros(NvS, dtype=np.int64)
        sel = (cp.dst_raw // NvS) == d
        np.add.at(hits, (cp.dst_raw[sel] % NvS), 1)
        assert hits.max() <= 1 and hits.sum() == N
        real = np.zeros(NvS, dtype=bool)
        start = 0
        for g in range(2 * epn):
            e = d * epn + g if g < epn else int(cp.experts_to_copy[d, g - epn])
            cnt = int(cp.alloc[e, d]) if e >= 0 else 0
            real[start:start + cnt] = True
            start = int(cu[g])
        assert (hits.astype(bool) == real).all(), "slots hit must be exactly the real rows"
