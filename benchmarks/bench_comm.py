"""Dispatch / combine micro-benchmark through the public Buffer API, swept over EP size,
hidden size, top-k and routing skew.

For every configuration it times the four operations a training step issues
(the same four the reference plots, benchmarks/bench_vs_deepep.py:186-232 there):

  dispatch_fwd   fresh dispatch: rank sync + planning + dispatch + duplicate expansion
  dispatch_bwd   dispatch with a saved plan (hidden only)
  combine_fwd    duplicate reduction + combine
  combine_bwd    the same with the [S, K] route-weight gather

Timing: by default ``--iters`` back-to-back calls are captured into one CUDA graph and the
replay is timed with CUDA events (no per-launch host cost on the timeline);
``--no-cudagraph`` times eager calls queued behind a device-side sleep instead, which keeps
every kernel a separate launch for profilers.  Reported per call, max over the ranks of the
EP group and over groups.  The hidden shard of every configuration in the default sweep is
larger than L2, so consecutive calls do not find their inputs in cache.

EP sizes smaller than the world run as disjoint sub-groups side by side (``Buffer(group=)``),
like the reference's sweep (benchmarks/bench_comm.py:529-536 there).

    python benchmarks/bench_comm.py                                   # one GPU, EP=1
    torchrun --nproc_per_node=8 benchmarks/bench_comm.py --ep 2 4 8 --out comm.csv
"""
import argparse
import csv
import itertools
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from moonep_b200 import Buffer, routing  # noqa: E402

OPS = ("dispatch_fwd", "dispatch_bwd", "combine_fwd", "combine_bwd")


def time_graph(fn, warmup, iters):
    """Per-call microseconds of ``fn`` replayed ``iters`` times from one CUDA graph."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(iters):
            fn()
    g.replay()                                  # first replay uploads the graph
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    g.replay()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e3 / iters


def time_eager(fn, warmup, iters):
    """Median microseconds of eager calls; a device-side sleep lets the host queue ahead."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    torch.cuda._sleep(400_000 * iters)
    for a, b in evs:
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    ts = sorted(a.elapsed_time(b) * 1e3 for a, b in evs)
    return ts[len(ts) // 2]


def run_config(ep, H, K, S, epn, mv, args, world, rank):
    """One configuration on every sub-group of size ``ep``; returns the result row on rank 0."""
    ngroups = world // ep
    groups = [dist.new_group(list(range(i * ep, (i + 1) * ep))) for i in range(ngroups)] if world > 1 else [None]
    if rank >= ngroups * ep:                    # leftover ranks idle for this configuration
        grp, grank = None, -1
    else:
        grp, grank = groups[rank // ep], rank % ep
    E = epn * ep
    row = {"ep": ep, "H": H, "K": K, "S": S, "E": E, "maxvio_target": mv, "num_sms": args.num_sms,
           "timing": "cudagraph" if args.cudagraph else "eager"}
    times = torch.zeros(len(OPS), device="cuda")
    stats = {}
    if grank >= 0:
        buf = Buffer(S, H, K, E, ep, num_sms=args.num_sms, token_padding=args.pad, group=grp)
        scale, _ = routing.solve_scale_for_maxvio(mv, S, K, E, ep, seed=0) if mv > 0 else (0.0, None)
        topk, w, tpe = (t.cuda() for t in routing.softmax_topk(S, K, E, scale, 0, grank))
        hidden = torch.randn(S, H, device="cuda").to(torch.bfloat16)
        _, _, _, plan = buf.dispatch(hidden, w, topk, tpe, zero_copy=True, router_weights_zero_copy=True)
        torch.cuda.synchronize()
        stats = buf.stats(plan)
        hv, wv = buf.hidden_nvsh_buffer_view, buf.router_weight_buffer_view
        fns = {
            "dispatch_fwd": lambda: buf.dispatch(hidden, w, topk, tpe, zero_copy=True, router_weights_zero_copy=True),
            "dispatch_bwd": lambda: buf.dispatch(hidden, plan=plan, zero_copy=True),
            "combine_fwd": lambda: buf.combine(plan=plan, hidden_nvsh=hv, zero_copy=True),
            "combine_bwd": lambda: buf.combine(plan=plan, hidden_nvsh=hv, route_weights_nvs=wv, zero_copy=True,
                                               router_weights_zero_copy=True),
        }
        timer = time_graph if args.cudagraph else time_eager
        for i, op in enumerate(OPS):
            times[i] = timer(fns[op], args.warmup, args.iters)
        buf.check()
        buf.destroy()
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        for g in groups:
            dist.destroy_process_group(g)
    payload = S * K * H * 2                     # logical bytes per rank, the reference's bandwidth convention
    for i, op in enumerate(OPS):
        row[op + "_us"] = round(float(times[i]), 1)
        row[op + "_logical_GBps"] = round(payload / max(float(times[i]), 1e-9) / 1e3, 1)
    row.update({k: (round(v, 4) if isinstance(v, float) else v) for k, v in stats.items()})
    return row


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ep", type=int, nargs="*", default=None, help="EP sizes (default: the world size)")
    ap.add_argument("--hidden", type=int, nargs="*", default=[7168])
    ap.add_argument("--topk", type=int, nargs="*", default=[8])
    ap.add_argument("--S", type=int, default=4096)
    ap.add_argument("--epn", type=int, default=32, help="experts per rank (E = epn * EP)")
    ap.add_argument("--experts", type=int, default=None, help="total experts E instead of --epn")
    ap.add_argument("--maxvio", type=float, nargs="*", default=[0.0, 1.0, 3.0])
    ap.add_argument("--num-sms", type=int, default=32)
    ap.add_argument("--pad", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--no-cudagraph", dest="cudagraph", action="store_false")
    ap.add_argument("--out", default=None, help="CSV path written by rank 0")
    ap.set_defaults(cudagraph=True)
    args = ap.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if world > 1:
        dist.init_process_group("nccl")
    eps = args.ep or [world]
    rows = []
    for ep, H, K, mv in itertools.product(eps, args.hidden, args.topk, args.maxvio):
        assert 1 <= ep <= world, f"--ep {ep} exceeds the world size {world}"
        epn = args.epn
        if args.experts is not None:
            assert args.experts % ep == 0, f"--experts {args.experts} is not a multiple of EP={ep}"
            epn = args.experts // ep
        row = run_config(ep, H, K, args.S, epn, mv, args, world, rank)
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
    if rank == 0 and args.out:
        keys = sorted({k for r in rows for k in r}, key=lambda k: (k not in ("ep", "H", "K", "S", "E"), k))
        with open(args.out, "w", newline="") as f:
            wr = csv.DictWriter(f, fieldnames=keys)
            wr.writeheader()
            wr.writerows(rows)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
