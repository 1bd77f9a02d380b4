"""Redundant-expert weight prefetch benchmark (``Buffer.prefetch_weight``).

One owner rank pushes its gate / up / down matrices into the spare slots of the ranks the
slot table names; a case is the fan-out of each of the owner's experts.  Reported per case:
median device time (max over ranks) and the owner's egress rate
``slots * 3 * H * H' * bytes / t``.  The payload of all but the smallest cases exceeds the
126 MB L2; ``--flush`` additionally rewrites a 256 MB buffer between timed launches.
Counterpart of the reference's benchmarks/bench_prefetch.py (same idea: fixed expert shape,
fan-out lists, bf16 and packed 8-bit payloads).

    torchrun --nproc_per_node=8 benchmarks/bench_prefetch.py
    python benchmarks/bench_prefetch.py --emulate-ranks 4        # one GPU, HBM-only figure
"""
import argparse
import json

import torch

from _pool_bench import PoolBench, cases_for, experts_to_copy_for, init_dist, time_launches

DTYPES = {"bf16": torch.bfloat16, "i8": torch.int8, "u8": torch.uint8}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--H", type=int, default=3584)
    ap.add_argument("--Hp", type=int, default=3072)
    ap.add_argument("--dtype", choices=sorted(DTYPES), default="bf16")
    ap.add_argument("--owner", type=int, default=0)
    ap.add_argument("--num-sms", type=int, default=32)
    ap.add_argument("--cases", nargs="*", default=None, help="labels to run (default: all)")
    ap.add_argument("--emulate-ranks", type=int, default=0)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--flush", action="store_true")
    args = ap.parse_args()

    world, rank = init_dist()
    R = args.emulate_ranks or world
    if R < 2:
        raise SystemExit("prefetch needs at least two ranks (torchrun, or --emulate-ranks R)")
    dtype = DTYPES[args.dtype]
    flush = torch.zeros(64 << 20, dtype=torch.float32, device="cuda") if args.flush else None
    benches = {}
    for case in cases_for(R, args.H, args.Hp):
        if args.cases and case["label"] not in args.cases:
            continue
        key = (case["epn"], case["H"], case["Hp"])
        if key not in benches:
            for b in benches.values():      # one set of pools alive at a time
                b.close()
            benches.clear()
            benches[key] = PoolBench(case["epn"], case["H"], case["Hp"], dtype, False, args.emulate_ranks, args.num_sms)
        pb = benches[key]
        etc = experts_to_copy_for(R, case["epn"], args.owner % R, case["counts"])
        plan = pb.plan(etc)
        us = pb.max_over_ranks(time_launches(lambda: pb.prefetch(plan), args.warmup, args.iters, flush))
        pb.check()
        slots = int((etc >= 0).sum())
        nbytes = slots * 3 * case["H"] * case["Hp"] * torch.tensor([], dtype=dtype).element_size()
        if rank == 0:
            print(json.dumps({"case": case["label"], "R": R, "epn": case["epn"], "H": case["H"], "Hp": case["Hp"],
                              "dtype": args.dtype, "slots": slots, "MB": round(nbytes / 1e6, 1),
                              "us": round(us, 1), "owner_egress_GBps": round(nbytes / us / 1e3, 1),
                              "emulated": bool(args.emulate_ranks), "num_sms": args.num_sms}))
    for b in benches.values():
        b.close()
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
