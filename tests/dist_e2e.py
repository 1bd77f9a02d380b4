"""Multi-process end-to-end scenario on real GPUs (one rank per GPU, VMM symmetric heap).

Run:  torchrun --nproc-per-node N --master-addr 127.0.0.1 --master-port P tests/dist_e2e.py
Every rank all-gathers the routing tables, solves the CPU oracle for the whole group and
checks its own plan, dispatched rows, combine result, prefetch slots and reduced grads.
Scenario follows the reference's tests/test_e2e.py:195-397 (sync vs async, plan reuse,
zero-copy aliasing, prefetch untouched when not requested, reduce_grad slot clearing).
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from moonep_b200 import Buffer, routing  # noqa: E402
from moonep_b200.pools import ExpertPools  # noqa: E402
from moonep_b200.sim import plan_cluster, dup_table_from_arrays, ops as simops  # noqa: E402
from gpu_helpers import traceable_hidden, defined_rows  # noqa: E402


class StageFailed(Exception):
    pass


ERRORS = []


def chk(cond, msg):
    if not bool(cond):
        ERRORS.append(str(msg))


def safe_check(buf):
    try:
        buf.check()
    except Exception as exc:  # a bounded wait expired on this rank: report it collectively
        ERRORS.append(f"{type(exc).__name__}: {exc}")


def stage(name):
    """Collective: every rank learns whether ANY rank failed a check, so that all of them stop
    together between steps (a rank must never exit while peers still touch its memory)."""
    torch.cuda.synchronize()
    ok = torch.tensor([0 if ERRORS else 1], device="cuda")
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if int(ok) == 0:
        raise StageFailed(name)


def main():
    dist.init_process_group("nccl")
    rank, R = dist.get_rank(), dist.get_world_size()
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    S, H, K, epn, pad = 256, 1024, 4, 8, 32
    E = R * epn
    Hp = 128
    # descriptor accounting: creating and destroying a Buffer (handle exchange over unix sockets,
    # imports, mappings) must leave no file descriptor open
    warm = Buffer(S, H, K, E, R, num_sms=16, token_padding=pad)     # first use opens library-internal files
    warm.destroy()
    fds_before = len(os.listdir("/proc/self/fd"))
    probe = Buffer(S, H, K, E, R, num_sms=16, token_padding=pad)
    probe.destroy()
    fds_after = len(os.listdir("/proc/self/fd"))
    chk(fds_after == fds_before, f"Buffer create + destroy leaked {fds_after - fds_before} file descriptors")
    buf = Buffer(S, H, K, E, R, num_sms=16, token_padding=pad)
    if rank == 0:
        print(f"[dist_e2e] multicast alias {'active' if buf._heap.mc_base else 'off'}", flush=True)
    pools = None
    try:
        pools = run_scenario(buf, rank, R, dev, S, H, K, epn, pad, E, Hp)
        failed = None
    except StageFailed as exc:
        failed = str(exc)
    # every rank reaches this point with no kernel in flight on any peer
    torch.cuda.synchronize()
    dist.barrier()
    if pools is not None:
        pools.destroy()
    buf.destroy()
    dist.barrier()
    if failed is not None:
        for e in ERRORS:
            print(f"[dist_e2e] rank {rank}: FAILED in stage '{failed}': {e}", flush=True)
        dist.destroy_process_group()
        sys.exit(1)
    if rank == 0:
        print(f"[dist_e2e] PASS on {R} ranks")
    dist.destroy_process_group()


def run_scenario(buf, rank, R, dev, S, H, K, epn, pad, E, Hp):

    topk_all = [routing.lognormal_topk(S, K, E, R, 1.5, 7, r)[0] for r in range(R)]
    cp = plan_cluster(np.stack([t.numpy() for t in topk_all]), E, pad)
    topk = topk_all[rank].to(dev)
    tpe = torch.bincount(topk.flatten().long(), minlength=E).to(torch.int32)
    hidden_all = [traceable_hidden(S, H, r) for r in range(R)]
    weights_all = [(torch.arange(S * K, dtype=torch.int32) + r * S * K + 1).view(torch.float32).reshape(S, K) for r in range(R)]
    hidden, weights = hidden_all[rank].to(dev), weights_all[rank].to(dev)

    # ---- fresh dispatch, sync
    h1, w1, cu1, plan1 = buf.dispatch(hidden, weights, topk, tpe)
    buf.verify_plan(plan1)            # replicated planners agree; every rank receives S*K rows
    torch.cuda.synchronize()
    safe_check(buf)
    chk(torch.equal(plan1.dst.cpu().long(), torch.from_numpy(cp.dst[rank])), "dst")
    chk(torch.equal(cu1.cpu().long(), torch.from_numpy(cp.cu_seqlens[rank])), "cu_seqlens")
    chk(torch.equal(plan1.experts_to_copy.cpu().long(), torch.from_numpy(cp.experts_to_copy)), "experts_to_copy")
    chk(torch.equal(plan1.remote_stats.cpu().long(), torch.from_numpy(cp.remote_stats[rank])), "remote_stats")
    got = dup_table_from_arrays(plan1.dup_groups.cpu().numpy(), plan1.dup_loffs.cpu().numpy(), plan1.dup_counts.cpu().numpy())
    chk(got == {k: tuple(sorted(v)) for k, v in cp.dup_tables[rank].items()}, "dup tables")
    eh, ew = simops.dispatch(cp, [h.view(torch.int16).float() for h in hidden_all],
                             [w.view(torch.int32).float() for w in weights_all], fill=-1.0)
    m = defined_rows(cp, rank)
    chk(torch.equal(h1.cpu().view(torch.int16).float()[m], eh[rank][m]), "dispatched rows")
    chk(torch.equal(w1.cpu().view(torch.int32).float()[m], ew[rank][m]), "dispatched weights")
    stage("fresh dispatch")
    snap = plan1.clone()

    # ---- async must equal sync
    h2, w2, cu2, plan2, ev = buf.dispatch(hidden, weights, topk, tpe, async_finish=True)
    ev.wait(torch.cuda.current_stream())
    torch.cuda.synchronize()
    chk(torch.equal(h2[m.to(dev)], h1[m.to(dev)]) and torch.equal(cu2, cu1) and torch.equal(plan2.dst, plan1.dst), 'torch.equal(h2[m.to(dev)], h1[m.to(dev)]) and torch.equal(cu')

    # ---- pools, prefetch (sync + async), untouched slots when not requested
    pools = ExpertPools(epn, (H, Hp), (H, Hp), (Hp, H), group=None, with_grads=True)
    ids = torch.arange(rank * epn, (rank + 1) * epn, device=dev, dtype=torch.float32).view(epn, 1, 1)
    for i, n in enumerate(("gate", "up", "down")):
        pools.local_weight(n).copy_((ids * 3 + i + torch.arange(pools.local_weight(n)[0].numel(), device=dev).view(pools.local_weight(n)[0].shape) % 5).to(torch.bfloat16))
        pools.prefetch_view(n)[rank].fill_(-9.0)
    torch.cuda.synchronize()
    dist.barrier()
    buf.prefetch_weight(plan=snap, **pools.prefetch_kwargs())
    torch.cuda.synchronize()
    safe_check(buf)
    dist.barrier()
    for i, n in enumerate(("gate", "up", "down")):
        shape = pools.local_weight(n)[0].shape
        for b in range(epn):
            e = int(cp.experts_to_copy[rank, b])
            slot = pools.prefetch_view(n)[rank, b]
            if e >= 0:
                want = (float(e) * 3 + i + torch.arange(slot.numel(), device=dev).view(shape) % 5).to(torch.bfloat16)
                chk(torch.equal(slot, want), f"{n}: slot {b} does not hold expert {e}")
            else:
                chk((slot == -9.0).all(), f"{n}: unused slot {b} was written")
    stage("prefetch")
    # compute view = [local | prefetch]
    cv = pools.compute_weight("gate")
    chk(cv.shape[0] == 2 * epn and cv[:epn].data_ptr() == pools.local_weight("gate").data_ptr(), 'cv.shape[0] == 2 * epn and cv[:epn].data_ptr() == pools.loca')
    chk(cv[epn:].data_ptr() == pools.prefetch_view("gate")[rank].data_ptr(), 'cv[epn:].data_ptr() == pools.prefetch_view("gate")[rank].dat')

    # ---- plan reuse (backward of combine): no planning, plan untouched
    before = snap.clone()
    hr, wr, cur, pr = buf.dispatch(hidden, plan=snap)
    torch.cuda.synchronize()
    chk(wr is None and cur is None and pr is snap, 'wr is None and cur is None and pr is snap')
    chk(torch.equal(hr[m.to(dev)], h1[m.to(dev)]), 'torch.equal(hr[m.to(dev)], h1[m.to(dev)])')
    for f in ("dst", "dup_groups", "dup_loffs", "dup_counts"):
        chk(torch.equal(getattr(snap, f), getattr(before, f)), 'torch.equal(getattr(snap, f), getattr(before, f))')
    stage("plan reuse")

    # ---- combine: identity FFN, zero-copy and copy paths agree; weights gather exact
    hz, wz, _, planz = buf.dispatch(hidden, weights, topk, tpe, zero_copy=True, router_weights_zero_copy=True)
    chk(hz.data_ptr() == buf.hidden_nvsh_buffer_view.data_ptr(), 'hz.data_ptr() == buf.hidden_nvsh_buffer_view.data_ptr()')
    oz, wsk, _ = buf.combine(plan=planz, hidden_nvsh=hz, route_weights_nvs=wz, zero_copy=True, router_weights_zero_copy=True)
    torch.cuda.synchronize()
    chk(torch.equal(wsk.view(torch.int32), weights.view(torch.int32)), "gathered weights")
    hc, wc, _, planc = buf.dispatch(hidden, weights, topk, tpe)
    oc, _, evc = buf.combine(plan=planc, hidden_nvsh=hc, async_finish=True)
    evc.wait(torch.cuda.current_stream())
    torch.cuda.synchronize()
    chk(torch.equal(oc, oz), "copy vs zero-copy combine")
    # numeric combine check with small integers
    y = torch.zeros(cp.NvS, H, dtype=torch.bfloat16)
    y[:] = ((torch.arange(cp.NvS) % 7) + 1 + rank)[:, None].to(torch.bfloat16)
    ys = []
    for r in range(R):
        t = torch.zeros(cp.NvS, H, dtype=torch.bfloat16)
        t[:] = ((torch.arange(cp.NvS) % 7) + 1 + r)[:, None].to(torch.bfloat16)
        ys.append(t.float())
    on, _, _ = buf.combine(plan=snap, hidden_nvsh=y.to(dev))
    torch.cuda.synchronize()
    eo, _ = simops.combine(cp, ys)
    chk(torch.equal(on.cpu().float(), eo[rank]), "combine sum")
    stage("combine")

    # ---- reduce_grad
    g = torch.Generator().manual_seed(11)
    lg_all = {n: [torch.randn(epn, *pools.shape(n), generator=g) for _ in range(R)] for n in ("gate", "up", "down")}
    rb_all = {n: [torch.randn(epn, *pools.shape(n), generator=g) for _ in range(R)] for n in ("gate", "up", "down")}
    for n in ("gate", "up", "down"):
        pools.local_grad(n).copy_(lg_all[n][rank])
        pools.reduce_view(n)[rank].copy_(rb_all[n][rank])
    torch.cuda.synchronize()
    dist.barrier()
    ev = buf.reduce_grad(plan=snap, async_finish=True, **pools.reduce_kwargs())
    ev.wait(torch.cuda.current_stream())
    torch.cuda.synchronize()
    safe_check(buf)
    dist.barrier()
    for n in ("gate", "up", "down"):
        el = [x.clone() for x in lg_all[n]]
        er = [x.clone() for x in rb_all[n]]
        simops.reduce_grad(cp, el, er)
        chk(torch.equal(pools.local_grad(n).cpu(), el[rank]), f"{n}: reduced grads (bitwise)")
        chk(torch.equal(pools.reduce_view(n)[rank].cpu(), er[rank]), f"{n}: reduce slots")
    stage("reduce_grad")

    # ---- repeated ops keep working (barrier epochs), then teardown
    for _ in range(3):
        buf.dispatch(hidden, weights, topk, tpe, zero_copy=True)
        buf.combine(plan=snap, hidden_nvsh=buf.hidden_nvsh_buffer_view, zero_copy=True)
    torch.cuda.synchronize()
    safe_check(buf)
    stage("repeat")
    symmetric_tensor_factories(rank, R, dev)
    return pools


def symmetric_tensor_factories(rank, R, dev):
    """The three tensor factories (all-rank view, multicast alias, single owner): every rank writes
    its own part, reads everybody else's and writes into the owner's memory."""
    from moonep_b200.parallel import create_dist_tensor, create_single_owner_tensor
    dt = create_dist_tensor((100, 48), torch.float32, multicast=True)
    chk(dt.local.shape == (100, 48) and dt.all.shape[0] == R * dt.rows, "dist tensor shapes")
    dt.local.fill_(float(rank + 1))
    torch.cuda.synchronize()
    dist.barrier()
    for r in range(R):
        chk(bool((dt.of_rank(r) == float(r + 1)).all()), f"dist tensor: chunk of rank {r} seen from rank {rank}")
    dt.of_rank((rank + 1) % R)[0, :].fill_(-float(rank + 1))        # a store into a peer's chunk
    torch.cuda.synchronize()
    dist.barrier()
    chk(bool((dt.local[0] == -float((rank - 1) % R + 1)).all()), "dist tensor: peer store landed")
    owner = R - 1
    so = create_single_owner_tensor((R, 64), torch.int32, owner=owner)
    chk(bool((so.tensor == 0).all()), "single-owner tensor starts zeroed")
    dist.barrier()
    so.tensor[rank].fill_(rank + 7)
    torch.cuda.synchronize()
    dist.barrier()
    want = (torch.arange(R, device=dev, dtype=torch.int32) + 7).unsqueeze(1).expand(R, 64)
    chk(torch.equal(so.tensor, want), "single-owner tensor: every rank's row visible everywhere")
    stage("symmetric tensor factories")
    so.destroy()
    dt.destroy()


if __name__ == "__main__":
    main()
