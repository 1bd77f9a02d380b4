"""Workload report of an EP configuration, computed on the CPU from the planner oracle.

For a group size, shape and routing skew it answers, without a GPU, the questions that size a
deployment: how many redundant experts the planner creates, which rank sends most, how many
bytes each collective moves over NVLink per rank and what that costs at a given link rate,
how many rows are duplicates (handled locally) and how many are padding.  The same counters
the reference's benchmark prints at run time (maxvio, dedup ratio, duplicate groups, padded
rows, GB/s; benchmarks/bench_comm.py:369-450 there), available before any hardware is booked.

    python -m moonep_b200.sim.report --R 8 --S 4096 --K 8 --E 256 --H 7168 --Hp 2048 --maxvio 0 1 3
"""

from __future__ import annotations

import argparse
import json

import numpy as np

from .. import routing
from .planner import plan_cluster


def workload(cp, H: int, Hp: int, link_gbps: float = 770.0) -> dict:
    """Counters of one cluster plan.  Bytes are per rank, for the busiest rank of each kind."""
    R, K, NvS, S = cp.R, cp.K, cp.NvS, cp.S
    epn = cp.E // R
    row = H * 2
    dest = cp.dst_raw // NvS                                   # [R, N]
    prim = cp.dst >= 0
    sent_remote = np.zeros(R, dtype=np.int64)                  # primary rows leaving rank r
    recv_remote = np.zeros(R, dtype=np.int64)
    for r in range(R):
        d = dest[r][prim[r]]
        remote = d[d != r]
        sent_remote[r] = remote.size
        recv_remote += np.bincount(remote, minlength=R)
    dup_rows = int((~prim).sum())
    total_rows = int(prim.size)
    distinct = prim.reshape(R, S, K).sum(axis=2).mean()        # distinct destination ranks per token
    etc = cp.experts_to_copy
    slots_recv = (etc >= 0).sum(axis=1)
    owner = np.where(etc >= 0, etc // epn, -1)
    slots_sent = np.array([(owner == r).sum() for r in range(R)])
    padded = int(cp.zero_fill_ranges[:, :, 1].sum())
    home = (np.arange(cp.E) // epn)[:, None] == np.arange(R)[None, :]
    moved = int(cp.alloc[~home].sum())                         # tokens computed away from their expert's home rank
    tot = cp.tpe.sum(axis=0).astype(np.float64)
    slot_w = 3 * H * Hp * 2                                    # gate + up + down, bf16
    out = {
        "maxvio": round(float(tot.max() / tot.mean() - 1.0), 3),
        "redundant_slots": int(slots_recv.sum()),
        "slots_sent_per_owner": slots_sent.tolist(),
        "max_slots_sent": int(slots_sent.max()), "max_slots_received": int(slots_recv.max()),
        "tokens_off_home_pct": round(100.0 * moved / max(1, int(cp.alloc.sum())), 2),
        "distinct_dest_ranks_per_token": round(float(distinct), 2),
        "duplicate_rows_pct": round(100.0 * dup_rows / total_rows, 1),
        "padded_rows_per_rank_max": int(cp.zero_fill_ranges[:, :, 1].sum(axis=1).max()),
        "padded_rows_total": padded,
        "NvS": NvS, "hidden_shard_MiB": round(NvS * row / 2**20, 1),
        "dispatch_egress_MB_max": round(float(sent_remote.max()) * row / 1e6, 1),
        "combine_ingress_MB_max": round(float(sent_remote.max()) * row / 1e6, 1),
        "dispatch_ingress_MB_max": round(float(recv_remote.max()) * row / 1e6, 1),
        "prefetch_egress_MB_max": round(float(slots_sent.max()) * slot_w / 1e6, 1),
        "grad_reduce_ingress_MB_max": round(float(slots_sent.max()) * slot_w * 2 / 1e6, 1),
    }
    us = lambda mb: round(mb * 1e6 / (link_gbps * 1e9) * 1e6, 1)  # noqa: E731
    out["link_GBps"] = link_gbps
    out["dispatch_us_at_link"] = us(max(out["dispatch_egress_MB_max"], out["dispatch_ingress_MB_max"]))
    out["combine_us_at_link"] = us(out["combine_ingress_MB_max"])
    out["prefetch_us_at_link"] = us(out["prefetch_egress_MB_max"])
    out["grad_reduce_us_at_link"] = us(out["grad_reduce_ingress_MB_max"])
    return out


def report(R: int, S: int, K: int, E: int, H: int, Hp: int, maxvio_target: float, token_padding: int = 128,
           seed: int = 0, link_gbps: float = 770.0) -> dict:
    scale, _ = routing.solve_scale_for_maxvio(maxvio_target, S, K, E, R, seed=seed) if maxvio_target > 0 else (0.0, None)
    topk = np.stack([routing.softmax_topk(S, K, E, scale, seed, r)[0].numpy() for r in range(R)])
    cp = plan_cluster(topk, E, token_padding)
    return {"R": R, "S": S, "K": K, "E": E, "H": H, "Hp": Hp, "maxvio_target": maxvio_target,
            "skew_scale": round(float(scale), 5), **workload(cp, H, Hp, link_gbps)}


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--R", type=int, default=8)
    ap.add_argument("--S", type=int, default=4096)
    ap.add_argument("--K", type=int, default=8)
    ap.add_argument("--E", type=int, default=256)
    ap.add_argument("--H", type=int, default=7168)
    ap.add_argument("--Hp", type=int, default=2048)
    ap.add_argument("--pad", type=int, default=128)
    ap.add_argument("--maxvio", type=float, nargs="*", default=[0.0, 1.0, 3.0])
    ap.add_argument("--link-gbps", type=float, default=770.0, help="NVLink rate per direction per GPU")
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args()
    for mv in a.maxvio:
        print(json.dumps(report(a.R, a.S, a.K, a.E, a.H, a.Hp, mv, a.pad, a.seed, a.link_gbps)))


if __name__ == "__main__":
    main()
