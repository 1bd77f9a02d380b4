"""Dispatch / combine / planning micro-benchmark through the public Buffer API.

Device-timed with CUDA events (max over ranks), warm-up first, L2 flushed between timed
iterations by the payload itself (the hidden shard is far larger than L2).  Mirrors what
the reference measures in benchmarks/bench_vs_deepep.py:186-232 (dispatch fwd incl.
planning, dispatch bwd with a saved plan, combine fwd, combine bwd with weight gather).

Launch: ``python benchmarks/bench_comm.py`` (1 GPU) or under torchrun for N ranks.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from moonep_b200 import Buffer, routing  # noqa: E402


def timed(fn, warmup, iters):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for a, b in evs:
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    ts = sorted(a.elapsed_time(b) * 1e3 for a, b in evs)
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--S", type=int, default=4096)
    ap.add_argument("--H", type=int, default=7168)
    ap.add_argument("--K", type=int, default=8)
    ap.add_argument("--epn", type=int, default=32)
    ap.add_argument("--num-sms", type=int, default=32)
    ap.add_argument("--pad", type=int, default=128)
    ap.add_argument("--maxvio", type=float, nargs="*", default=[0.0, 1.0, 3.0])
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if world > 1:
        dist.init_process_group("nccl")
    R, E = world, args.epn * world
    buf = Buffer(args.S, args.H, args.K, E, R, num_sms=args.num_sms, token_padding=args.pad)
    rows = []
    for mv in args.maxvio:
        scale, realised = routing.solve_scale_for_maxvio(mv, args.S, args.K, E, R, seed=0) if mv > 0 else (0.0, None)
        topk, w, tpe = routing.softmax_topk(args.S, args.K, E, scale, 0, rank)
        topk, w, tpe = topk.cuda(), w.cuda(), tpe.cuda()
        hidden = torch.randn(args.S, args.H, device="cuda").to(torch.bfloat16)
        h, wn, cu, plan = buf.dispatch(hidden, w, topk, tpe, zero_copy=True, router_weights_zero_copy=True)
        torch.cuda.synchronize()
        res = {"maxvio_target": mv, "scale": scale, **buf.stats(plan)}
        res["dispatch_fwd_us"] = timed(lambda: buf.dispatch(hidden, w, topk, tpe, zero_copy=True, router_weights_zero_copy=True), args.warmup, args.iters)
        res["dispatch_bwd_us"] = timed(lambda: buf.dispatch(hidden, plan=plan, zero_copy=True), args.warmup, args.iters)
        hv, wv = buf.hidden_nvsh_buffer_view, buf.router_weight_buffer_view
        res["combine_fwd_us"] = timed(lambda: buf.combine(plan=plan, hidden_nvsh=hv, zero_copy=True), args.warmup, args.iters)
        res["combine_bwd_us"] = timed(lambda: buf.combine(plan=plan, hidden_nvsh=hv, route_weights_nvs=wv, zero_copy=True, router_weights_zero_copy=True), args.warmup, args.iters)
        if world > 1:
            for k in [k for k in res if k.endswith("_us")]:
                t = torch.tensor([res[k]], device="cuda")
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                res[k] = float(t)
        buf.check()
        rows.append(res)
        if rank == 0:
            print(json.dumps(res))
    buf.destroy()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
