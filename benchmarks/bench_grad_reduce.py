"""Redundant-expert gradient reduction benchmark (``Buffer.reduce_grad``).

The owner of replicated experts pulls the fp32 partial gradients out of every holder's
reduce slots, adds them to its local gradients in slot order, and each holder clears the
slots it lent -- one launch for gate, up and down.  A case is the fan-out of each of the
owner's experts.  Reported per case: median device time (max over ranks) and the owner's
ingress rate ``slots * 3 * H * H' * 4 / t``.  Counterpart of the reference's
benchmarks/bench_grad_reduce.py, which times its three per-projection launches.

    torchrun --nproc_per_node=8 benchmarks/bench_grad_reduce.py
    python benchmarks/bench_grad_reduce.py --emulate-ranks 4     # one GPU, HBM-only figure
"""
import argparse
import json

import torch

from _pool_bench import PoolBench, cases_for, experts_to_copy_for, init_dist, time_launches


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--H", type=int, default=3584)
    ap.add_argument("--Hp", type=int, default=3072)
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
        raise SystemExit("reduce_grad needs at least two ranks (torchrun, or --emulate-ranks R)")
    flush = torch.zeros(64 << 20, dtype=torch.float32, device="cuda") if args.flush else None
    pb, key = None, None
    for case in cases_for(R, args.H, args.Hp):
        if args.cases and case["label"] not in args.cases:
            continue
        k = (case["epn"], case["H"], case["Hp"])
        if k != key:
            if pb is not None:
                pb.close()
            pb, key = PoolBench(case["epn"], case["H"], case["Hp"], torch.bfloat16, True, args.emulate_ranks,
                                args.num_sms), k
        etc = experts_to_copy_for(R, case["epn"], args.owner % R, case["counts"])
        plan = pb.plan(etc)
        # the kernel clears the consumed slots, so every launch sees zeros after the first:
        # the traffic is the same, the values are irrelevant to the timing
        us = pb.max_over_ranks(time_launches(lambda: pb.reduce_grad(plan), args.warmup, args.iters, flush))
        pb.check()
        slots = int((etc >= 0).sum())
        nbytes = slots * 3 * case["H"] * case["Hp"] * 4
        if rank == 0:
            print(json.dumps({"case": case["label"], "R": R, "epn": case["epn"], "H": case["H"], "Hp": case["Hp"],
                              "slots": slots, "MB": round(nbytes / 1e6, 1), "us": round(us, 1),
                              "owner_ingress_GBps": round(nbytes / us / 1e3, 1),
                              "emulated": bool(args.emulate_ranks), "num_sms": args.num_sms}))
    if pb is not None:
        pb.close()
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
