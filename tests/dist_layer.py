"""Multi-process check of the fused MoE layer on real GPUs (one rank per GPU, peer memory over
NVLink): ``ExpertParallelMoE`` forward and backward against a dense fp32 implementation of the same
top-k MoE built from all-gathered inputs and weights.

Run:  torchrun --nproc-per-node N --master-addr 127.0.0.1 --master-port P tests/dist_layer.py
Variants: push-combine on / off (peer stores from the down GEMM's epilogue), tile-ready flags on /
off (GEMMs that consume the shard while the dispatch kernel is still receiving), backward overlap on /
off (split launches beside the communication kernels).  Routing is skewed so that the planner creates
redundant experts (prefetch + cross-rank gradient reduction are exercised).
Counterpart of the reference's public-API scenario tests/test_e2e.py:195-397, one level up: through the
layer that integrates the API with the expert GEMMs.  A failed check is agreed on collectively between
variants, so no rank leaves while a peer still touches its memory.
"""
import itertools
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from moonep_b200 import Buffer, routing  # noqa: E402
from moonep_b200.moe_layer import ExpertParallelMoE, moe_apply  # noqa: E402
from moonep_b200.ops import grouped_gemm as gg  # noqa: E402
from moonep_b200.pools import ExpertPools  # noqa: E402

ERRORS = []


def chk(cond, msg):
    if not bool(cond):
        ERRORS.append(str(msg))


def agree(name):
    """Collective: True if no rank has recorded an error so far."""
    torch.cuda.synchronize()
    ok = torch.tensor([0 if ERRORS else 1], device="cuda")
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    return int(ok) == 1


def gather(t):
    out = [torch.empty_like(t) for _ in range(dist.get_world_size())]
    dist.all_gather(out, t.contiguous())
    return out


def rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


def dense_reference(xs, ws, topks, gys, Wg, Wu, Wd, rank, epn):
    """fp32 MoE over ALL ranks' tokens; returns this rank's output, input grad, route-weight grad and the
    weight grads of its own experts."""
    R = len(xs)
    X = [x.float().requires_grad_(True) for x in xs]
    Wt = [w.clone().requires_grad_(True) for w in ws]
    Wg, Wu, Wd = (t.float().requires_grad_(True) for t in (Wg, Wu, Wd))
    outs = []
    for r in range(R):
        y = torch.zeros_like(X[r])
        for k in range(topks[r].shape[1]):
            e = topks[r][:, k].long()
            h = torch.nn.functional.silu(torch.einsum("sh,shp->sp", X[r], Wg[e])) * torch.einsum("sh,shp->sp", X[r], Wu[e])
            y = y + Wt[r][:, k:k + 1] * torch.einsum("sp,sph->sh", h, Wd[e])
        outs.append(y)
    torch.autograd.backward(outs, [g.float() for g in gys])
    sl = slice(rank * epn, (rank + 1) * epn)
    return outs[rank].detach(), X[rank].grad, Wt[rank].grad, Wg.grad[sl], Wu.grad[sl], Wd.grad[sl]


def shared_slots_scenario(rank, R, dev):
    """Two layers with different experts share ONE Buffer and ONE set of prefetch / reduce slots
    (``pools.SharedSlots``): forward A, forward B, backward B, backward A.  By the time a layer runs its
    backward pass the slots hold the other layer's experts, so it must fetch its own again; each layer is
    compared with its own dense reference."""
    from moonep_b200.pools import SharedSlots
    S, H, Hp, K, epn, pad = 256, 512, 512, 4, 4, 128        # 4 x 512 x 512 bf16 = one mapping granule per projection
    E = R * epn
    gen = torch.Generator(device=dev).manual_seed(500 + rank)
    buf = Buffer(S, H, K, E, R, num_sms=8, token_padding=pad, push_combine=True)
    shared = SharedSlots(epn, (H, Hp), (H, Hp), (Hp, H), with_grads=True)
    layers = []
    for li in range(2):
        topk = routing.lognormal_topk(S, K, E, R, 1.2, 11 + li, rank)[0].to(dev)
        tpe = torch.bincount(topk.flatten().long(), minlength=E).to(torch.int32)
        x0 = (torch.randn(S, H, device=dev, generator=gen) * 0.5).to(torch.bfloat16)
        w0 = torch.rand(S, K, device=dev, generator=gen) + 0.1
        w0 = (w0 / w0.sum(dim=1, keepdim=True)).contiguous()
        gy = (torch.randn(S, H, device=dev, generator=gen) * 0.1).to(torch.bfloat16)
        lw = {n: (torch.randn(epn, *shp, device=dev, generator=gen) * 0.04).to(torch.bfloat16)
              for n, shp in (("gate", (H, Hp)), ("up", (H, Hp)), ("down", (Hp, H)))}
        allw = {n: torch.cat(gather(t)) for n, t in lw.items()}
        want = dense_reference(gather(x0), gather(w0), gather(topk), gather(gy), allw["gate"], allw["up"], allw["down"], rank, epn)
        pools = ExpertPools(epn, (H, Hp), (H, Hp), (Hp, H), with_grads=True, shared=shared)
        for n in ("gate", "up", "down"):
            pools.local_weight(n).copy_(lw[n])
            pools.compute_grad(n).zero_()
        layers.append(dict(topk=topk, tpe=tpe, x0=x0, w0=w0, gy=gy, want=want, pools=pools,
                           moe=ExpertParallelMoE(buf, pools)))
    torch.cuda.synchronize()
    dist.barrier()
    for rep in range(2):
        ys = []
        for L in layers:
            L["x"], L["w"] = L["x0"].clone().requires_grad_(True), L["w0"].clone().requires_grad_(True)
            ys.append(moe_apply(L["moe"], L["x"], L["w"], L["topk"], L["tpe"]))
        for L, y in reversed(list(zip(layers, ys))):
            y.backward(L["gy"])
            L["moe"].wait_grads()
        torch.cuda.synchronize()
        try:
            buf.check()
            gg.check_status()
        except Exception as exc:      # noqa: BLE001
            ERRORS.append(f"shared slots: {type(exc).__name__}: {exc}")
        for li, (L, y) in enumerate(zip(layers, ys)):
            p = L["pools"]
            got = (y, L["x"].grad, L["w"].grad, p.local_grad("gate"), p.local_grad("up"), p.local_grad("down"))
            for label, a, b in zip(("output", "grad hidden", "grad route weights", "grad gate", "grad up", "grad down"), got, L["want"]):
                chk(torch.isfinite(a.float()).all() and rel(a, b) < 3e-2, f"shared slots, layer {li} rep {rep}: {label} off by {rel(a, b):.4f}")
    ok = agree("shared slots")
    if rank == 0:
        print(f"[dist_layer] two layers on one Buffer and one set of slots: {'ok' if ok else 'FAILED'}", flush=True)
    torch.cuda.synchronize()
    dist.barrier()
    for L in layers:
        L["pools"].destroy()
    shared.destroy()
    buf.destroy()
    dist.barrier()


def epilogue_optimizer_scenario(rank, R, dev):
    """Two training steps with the SGD update inside the weight-gradient GEMMs' epilogue (experts without
    replicas) plus the stored-gradient path for replicated experts, against the same two steps
    with the stand-alone optimizer after the backward pass: the weights must come out bit for bit equal."""
    S, H, Hp, K, epn, pad, lr = 256, 256, 256, 4, 4, 128, 0.5
    E = R * epn
    topk = routing.lognormal_topk(S, K, E, R, 1.2, 3, rank)[0].to(dev)
    tpe = torch.bincount(topk.flatten().long(), minlength=E).to(torch.int32)
    g = torch.Generator(device=dev).manual_seed(300 + rank)
    x0 = (torch.randn(S, H, device=dev, generator=g) * 0.5).to(torch.bfloat16)
    w0 = torch.rand(S, K, device=dev, generator=g) + 0.1
    w0 = (w0 / w0.sum(dim=1, keepdim=True)).contiguous()
    gy = (torch.randn(S, H, device=dev, generator=g) * 0.1).to(torch.bfloat16)
    init = {n: (torch.randn(epn, *shp, device=dev, generator=g) * 0.05).to(torch.bfloat16)
            for n, shp in (("gate", (H, Hp)), ("up", (H, Hp)), ("down", (Hp, H)))}
    final, fused_any = [], 0
    for in_epilogue, overlap in ((False, True), (True, True), (True, False)):
        buf = Buffer(S, H, K, E, R, num_sms=8, token_padding=pad, push_combine=True)
        pools = ExpertPools(epn, (H, Hp), (H, Hp), (Hp, H), with_grads=True)
        for n in init:
            pools.local_weight(n).copy_(init[n])
            pools.compute_grad(n).zero_()
        torch.cuda.synchronize()
        dist.barrier()
        layer = ExpertParallelMoE(buf, pools, overlap_backward=overlap, ready_flags=True)
        layer.defer_last_reduction = True        # the reduction of ``up`` (and the update behind it) is joined by wait_grads()
        if in_epilogue:
            layer.epilogue_lr = lr

            def rest(n, layer=layer, pools=pools):
                gg.sgd_step_groups(pools.local_weight(n), pools.local_grad(n), lr, layer._upd_mask, want=False)
            layer.on_grad_ready = rest
        for rep in range(2):
            x = x0.clone().requires_grad_(True)
            w = w0.clone().requires_grad_(True)
            y = moe_apply(layer, x, w, topk, tpe)
            y.backward(gy)
            layer.wait_grads()
            if not in_epilogue:
                for n in init:
                    gg.sgd_step(pools.local_weight(n), pools.local_grad(n), lr)
            torch.cuda.synchronize()
            dist.barrier()          # every owner has updated before anyone prefetches its experts again
        try:
            buf.check()
            gg.check_status()
        except Exception as exc:      # noqa: BLE001
            ERRORS.append(f"epilogue optimizer ({in_epilogue}): {type(exc).__name__}: {exc}")
        if in_epilogue:
            fused_any = int(layer._upd_mask[:epn].sum())
        final.append({n: pools.local_weight(n).clone() for n in init})
        torch.cuda.synchronize()
        dist.barrier()
        pools.destroy()
        buf.destroy()
        dist.barrier()
    for n in init:
        chk(not torch.equal(final[0][n], init[n]), f"epilogue optimizer: {n} was not trained")
        for v, label in ((1, "overlapped backward"), (2, "serial backward")):
            chk(torch.equal(final[0][n], final[v][n]),
                f"epilogue optimizer, {label}: {n} differs from the stand-alone optimizer "
                f"({int((final[0][n] != final[v][n]).sum())} elements)")
    tot = torch.tensor([fused_any, epn - fused_any], device=dev)
    dist.all_reduce(tot)
    chk(int(tot[0]) > 0, "epilogue optimizer: no expert took the fused path")
    chk(int(tot[1]) > 0 or R == 1, "epilogue optimizer: no expert took the stored-gradient path")
    ok = agree("epilogue optimizer")
    if rank == 0:
        print(f"[dist_layer] optimizer in the weight-gradient epilogue ({int(tot[0])} experts fused, {int(tot[1])} reduced first): "
              f"{'ok' if ok else 'FAILED'}", flush=True)


def main():
    dist.init_process_group("nccl")
    rank, R = dist.get_rank(), dist.get_world_size()
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    S, H, Hp, K, epn, pad = 256, 256, 256, 4, 4, 128
    E = R * epn
    topk = routing.lognormal_topk(S, K, E, R, 1.2, 3, rank)[0].to(dev)
    tpe = torch.bincount(topk.flatten().long(), minlength=E).to(torch.int32)
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    x0 = (torch.randn(S, H, device=dev, generator=g) * 0.5).to(torch.bfloat16)
    w0 = torch.rand(S, K, device=dev, generator=g) + 0.1
    w0 = (w0 / w0.sum(dim=1, keepdim=True)).contiguous()
    gy = (torch.randn(S, H, device=dev, generator=g) * 0.1).to(torch.bfloat16)
    local_w = {n: (torch.randn(epn, *shp, device=dev, generator=g) * 0.05).to(torch.bfloat16)
               for n, shp in (("gate", (H, Hp)), ("up", (H, Hp)), ("down", (Hp, H)))}
    xs, ws, topks, gys = gather(x0), gather(w0), gather(topk), gather(gy)
    allw = {n: torch.cat(gather(t)) for n, t in local_w.items()}
    want = dense_reference(xs, ws, topks, gys, allw["gate"], allw["up"], allw["down"], rank, epn)
    redundancy_seen = False

    variants = list(itertools.product((False, True), (False, True), (False, True)))     # push, flags, overlap
    for push, flags, overlap in variants:
        name = f"push={int(push)} flags={int(flags)} overlap={int(overlap)}"
        buf = Buffer(S, H, K, E, R, num_sms=8, token_padding=pad, push_combine=push)
        pools = ExpertPools(epn, (H, Hp), (H, Hp), (Hp, H), with_grads=True)
        for n in ("gate", "up", "down"):
            pools.local_weight(n).copy_(local_w[n])
            pools.compute_grad(n).zero_()
        torch.cuda.synchronize()
        dist.barrier()
        layer = ExpertParallelMoE(buf, pools, overlap_backward=overlap, ready_flags=flags)
        for rep in range(2):            # twice: barrier epochs, flag epochs and ticket counters carry over
            x = x0.clone().requires_grad_(True)
            w = w0.clone().requires_grad_(True)
            y = moe_apply(layer, x, w, topk, tpe)
            y.backward(gy)
            layer.wait_grads()
            torch.cuda.synchronize()
            try:
                buf.check()
                gg.check_status()
            except Exception as exc:      # noqa: BLE001
                ERRORS.append(f"{name}: {type(exc).__name__}: {exc}")
            got = (y, x.grad, w.grad, pools.local_grad("gate"), pools.local_grad("up"), pools.local_grad("down"))
            for label, a, b, tol in zip(("output", "grad hidden", "grad route weights", "grad gate", "grad up", "grad down"),
                                        got, want, (2e-2, 3e-2, 3e-2, 3e-2, 3e-2, 3e-2)):
                chk(torch.isfinite(a.float()).all(), f"{name} rep {rep}: {label} is not finite")
                chk(rel(a, b) < tol, f"{name} rep {rep}: {label} off by {rel(a, b):.4f}")
        if not redundancy_seen:
            c = buf.counters()
            sent = torch.tensor([c.get("rows_sent_remote", 0)], device=dev)
            dist.all_reduce(sent)
            chk(int(sent) > 0 or R == 1, "no row crossed a link")
            redundancy_seen = True
        ok = agree(name)
        if rank == 0:
            print(f"[dist_layer] {name}: {'ok' if ok else 'FAILED'}", flush=True)
        torch.cuda.synchronize()
        dist.barrier()
        pools.destroy()
        buf.destroy()
        dist.barrier()
        if not ok and any("Timeout" in e or "aborted" in e for e in ERRORS):
            break           # a device-side wait ran out: later variants would only repeat it
    if not ERRORS:
        shared_slots_scenario(rank, R, dev)
    if not ERRORS:
        epilogue_optimizer_scenario(rank, R, dev)
    if ERRORS:
        for e in ERRORS[:24]:
            print(f"[dist_layer] rank {rank}: {e}", flush=True)
    failed = not agree("end")
    dist.destroy_process_group()
    if failed:
        sys.exit(1)
    if rank == 0:
        print(f"[dist_layer] PASS on {R} ranks")


if __name__ == "__main__":
    main()
