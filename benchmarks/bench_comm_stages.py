"""Per-kernel device times of the communication path (planning, dispatch, duplicate finalize /
expand / reduce, combine, prefetch, grad_reduce), CUDA events, median over iterations, max
over ranks.  1 GPU: ``python benchmarks/bench_comm_stages.py``; N GPUs: under torchrun.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from moonep_b200 import Buffer, engine, routing  # noqa: E402
from moonep_b200.pools import ExpertPools  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--S", type=int, default=4096)
    ap.add_argument("--H", type=int, default=7168)
    ap.add_argument("--Hp", type=int, default=2048)
    ap.add_argument("--K", type=int, default=8)
    ap.add_argument("--epn", type=int, default=32)
    ap.add_argument("--num-sms", type=int, default=32)
    ap.add_argument("--maxvio", type=float, default=1.0)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--pools", action="store_true", help="also time prefetch and grad_reduce")
    a = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1")); rank = int(os.environ.get("RANK", "0"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if world > 1:
        dist.init_process_group("nccl")
    R, E = world, a.epn * world
    buf = Buffer(a.S, a.H, a.K, E, R, num_sms=a.num_sms)
    st = buf._states
    scale, _ = routing.solve_scale_for_maxvio(a.maxvio, a.S, a.K, E, R, seed=0) if a.maxvio > 0 else (0.0, 0)
    topk, w, tpe = (t.cuda() for t in routing.softmax_topk(a.S, a.K, E, scale, 0, rank))
    hidden = torch.randn(a.S, a.H, device="cuda").to(torch.bfloat16)
    plan, cu = engine.allocate_plan(st[0], with_send_list=True)
    out = torch.empty(a.S, a.H, dtype=torch.bfloat16, device="cuda")
    outw = torch.empty(a.S, a.K, device="cuda")
    nd = buf._num_sms_dedup * 4
    stages = [
        ("planning", lambda: engine.launch_planning(st, [topk.reshape(-1)], [tpe], [plan], [cu])),
        ("dispatch", lambda: engine.launch_dispatch(st, [hidden], [w], [plan], fresh=True, entry_barrier=False)),
        ("dup_finalize", lambda: engine.launch_dup_finalize(st, [plan])),
        ("dup_expand", lambda: engine.launch_dup_expand(st, [st[0].hidden_local], [plan], nd)),
        ("dup_reduce", lambda: engine.launch_dup_reduce(st, [st[0].hidden_local], [plan], nd)),
        ("combine", lambda: engine.launch_combine(st, [plan], [out], [outw], entry_barrier=True)),
        # flagged path: send list, then the slot-ordered dispatch that also expands duplicate rows
        ("send_order", lambda: engine.launch_send_order(st, [plan], [cu])),
        ("dispatch_flagged", lambda: (engine.launch_flag_epoch_bump(st),
                                      engine.launch_dispatch(st, [hidden], [w], [plan], fresh=True, entry_barrier=False, flagged=True))),
    ]
    pools = None
    if a.pools and world > 1:
        pools = ExpertPools(a.epn, (a.H, a.Hp), (a.H, a.Hp), (a.Hp, a.H), with_grads=True)
        pk = pools.prefetch_kwargs(); rk = pools.reduce_kwargs()
        pw = [(pk[f"local_{n}_weight"], pk[f"{n}_prefetch_buffer"]) for n in ("gate", "up", "down")]
        rg = [(rk[f"local_{n}_grad"], rk[f"{n}_reduce_buffer"]) for n in ("gate", "up", "down")]
        stages += [("prefetch", lambda: engine.launch_prefetch(st, [plan.experts_to_copy], [pw])),
                   ("grad_reduce", lambda: engine.launch_grad_reduce(st, [plan.experts_to_copy], [rg]))]
    times = {n: [] for n, _ in stages}
    for it in range(a.iters + 2):
        for name, fn in stages:
            if world > 1:
                dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record()
            torch.cuda.synchronize()
            if it >= 2:
                times[name].append(e0.elapsed_time(e1) * 1e3)
    buf.check()
    res = {"n_gpus": world, "maxvio": a.maxvio, **buf.stats(plan)}
    for name in times:
        t = sorted(times[name])[len(times[name]) // 2]
        if world > 1:
            tt = torch.tensor([t], device="cuda"); dist.all_reduce(tt, op=dist.ReduceOp.MAX); t = float(tt)
        res[name + "_us"] = round(t, 1)
    if rank == 0:
        print(json.dumps(res))
    if pools is not None:
        pools.destroy()
    buf.destroy()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
