"""Reference arm: the same MoE-layer training step as bench.py, but every communication op
goes through the UNMODIFIED reference package's public API (``moonep.Buffer``: dispatch,
prefetch_weight, combine, reduce_grad) and the expert FFN -- which the reference leaves to the
integrating framework -- is written the way an integrator without a grouped-GEMM library would:
library GEMMs (either ``torch._grouped_mm`` driven by the device-side ``cu_seqlens``, or one cuBLAS
``torch.mm`` per expert group writing straight into preallocated activations and, in fp32, into the
weight-gradient views; the faster of the two is picked during warm-up), SwiGLU forward / backward
and the SGD update as single fused element-wise kernels (``torch.compile``, eager if that is not
available).  Nothing of ``moonep_b200`` runs here.  Same shapes, routing generator, loss,
optimizer step, timing rules and JSON line as the main arm.
Imported only by bench_reference.py after ``baseline/_ref`` has been put on ``sys.path``.
"""

import json
import os
import sys
import time

import torch
import torch.distributed as dist

from benchmarks._loss import mean_square

CFG = {"deepseek_v3": dict(H=7168, Hp=2048, K=8, epn=32, S=4096),
       "qwen3_30b_a3b": dict(H=2048, Hp=768, K=8, epn=16, S=8192)}
SWEEP = (0.0, 0.5, 1.0, 2.0, 3.0)


def _gmm(a, b, offs):
    """a [M, K] x b [G, K, N] grouped by row offsets -> [M, N] (rows past offs[-1] undefined)."""
    if hasattr(torch, "_grouped_mm"):
        return torch._grouped_mm(a, b, offs=offs)
    out = torch.zeros(a.shape[0], b.shape[2], dtype=a.dtype, device=a.device)
    s = 0
    for g, e in enumerate(offs.tolist()):
        if e > s:
            out[s:e] = a[s:e] @ b[g]
        s = e
    return out


def _gmm_wgrad(x, dy, offs, G):
    """per group x_g^T dy_g -> [G, K, N]."""
    if hasattr(torch, "_grouped_mm"):
        return torch._grouped_mm(x.t(), dy, offs=offs)
    out = torch.zeros(G, x.shape[1], dy.shape[1], dtype=x.dtype, device=x.device)
    s = 0
    for g, e in enumerate(offs.tolist()):
        if e > s:
            out[g] = x[s:e].t() @ dy[s:e]
        s = e
    return out


def _clock_sampler(local_rank):
    """nvidia-smi sampler of the clocks during the timed region.  The class is loaded from its source
    file (standard library only), so that the package with the kernels is not imported on this path."""
    import importlib.util
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "moonep_b200", "utils", "clocks.py")
    try:
        spec = importlib.util.spec_from_file_location("_mep_clocks", path)
        mod = importlib.util.module_from_spec(spec)
        sys.modules["_mep_clocks"] = mod
        spec.loader.exec_module(mod)
        return mod.ClockSampler(local_rank).start()
    except Exception:      # noqa: BLE001
        return None


def run(args):
    from moonep import Buffer
    from moonep.buffer import create_nvl_dist_tensor

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    dist.init_process_group("nccl")
    dev = torch.device("cuda", local)
    c = CFG[args.model]
    S, H, Hp, K, epn = c["S"], c["H"], c["Hp"], c["K"], c["epn"]
    E, R = epn * world, world
    buffer = Buffer(S=S, H=H, K=K, E=E, num_ep_ranks=R, num_sms=32, token_padding=128)

    def pool(rows, cols, dtype):
        t = create_nvl_dist_tensor([2 * epn, rows, cols], dtype, rank, R)
        return t.view(R, 2 * epn, rows, cols)

    g = torch.Generator(device=dev).manual_seed(rank)
    shapes = {"gate": (H, Hp), "up": (H, Hp), "down": (Hp, H)}
    W, Gd = {}, {}
    for n, (r_, c_) in shapes.items():
        W[n] = pool(r_, c_, torch.bfloat16)
        W[n][rank, :epn].copy_((torch.randn(epn, r_, c_, device=dev, generator=g) * 0.02).to(torch.bfloat16))
        Gd[n] = pool(r_, c_, torch.float32)
        Gd[n][rank].zero_()
    gs = torch.Generator(device=dev).manual_seed(0)
    router = (torch.randn(H, E, device=dev, generator=gs) * 0.02).to(torch.bfloat16).requires_grad_(True)
    bias_base = torch.randn(E, device=dev, generator=torch.Generator(device=dev).manual_seed(1234)).float()
    state = {"bias": bias_base * 0.0}
    torch.cuda.synchronize()
    dist.barrier()

    def route(x):
        logits = (x @ router).float() + state["bias"]
        probs = torch.softmax(logits, dim=-1)
        w, topk = torch.topk(probs, K, dim=-1)
        w = (w / w.sum(dim=-1, keepdim=True)).contiguous()
        topk = topk.to(torch.int32).contiguous()
        tpe = torch.zeros(E, dtype=torch.int32, device=dev)
        tpe.scatter_add_(0, topk.reshape(-1).long(), torch.ones(topk.numel(), dtype=torch.int32, device=dev))
        return w, topk, tpe

    def prefetch_kwargs():
        kw = {}
        for n in shapes:
            kw[f"local_{n}_weight"] = W[n][rank, :epn]
            kw[f"{n}_prefetch_buffer"] = W[n][:, epn:]
        return kw

    def reduce_kwargs():
        kw = {}
        for n in shapes:
            kw[f"local_{n}_grad"] = Gd[n][rank, :epn]
            kw[f"{n}_reduce_buffer"] = Gd[n][:, epn:]
        return kw

    NvS = buffer.NvS if hasattr(buffer, "NvS") else None
    ffn = {"mode": os.environ.get("MOONEP_REF_FFN", "grouped")}      # "grouped" | "loop", settled in the warm-up

    # ---- fused element-wise pieces (one kernel each when torch.compile works on this machine)
    def _swiglu_fwd(gp, up, w):
        g = gp.float()
        return (torch.nn.functional.silu(g) * up.float() * w[:, None]).to(torch.bfloat16)

    def _swiglu_bwd(dA, gp, up, w):
        dAf, gf, uf = dA.float(), gp.float(), up.float()
        sig = torch.sigmoid(gf)
        silu = gf * sig
        dw = (dAf * silu * uf).sum(dim=1)
        d = dAf * w[:, None]
        dg = (d * uf * sig * (1 + gf * (1 - sig))).to(torch.bfloat16)
        du = (d * silu).to(torch.bfloat16)
        return dg, du, dw

    def _sgd(p, g, lr_):
        p.copy_((p.float() - lr_ * g).to(torch.bfloat16))

    fused = {"fwd": _swiglu_fwd, "bwd": _swiglu_bwd, "sgd": _sgd, "how": "eager"}
    if os.environ.get("MOONEP_REF_COMPILE", "1") != "0":
        try:
            cf, cb, cs = torch.compile(_swiglu_fwd), torch.compile(_swiglu_bwd), torch.compile(_sgd)
            t = torch.randn(256, 128, device=dev).to(torch.bfloat16)
            ww = torch.rand(256, device=dev)
            cf(t, t, ww); cb(t, t, t, ww)
            pp = torch.zeros(64, 64, device=dev, dtype=torch.bfloat16)
            cs(pp, torch.zeros(64, 64, device=dev), 1e-3)
            torch.cuda.synchronize()
            fused = {"fwd": cf, "bwd": cb, "sgd": cs, "how": "torch.compile"}
        except Exception:      # noqa: BLE001  (no compiler toolchain for the generated kernels: stay eager)
            pass

    def _segments(cu):
        """Non-empty (group, begin, end) row ranges; one host read of cu_seqlens per layer pass."""
        out, beg = [], 0
        for gidx, end in enumerate(cu.tolist()):
            if end > beg:
                out.append((gidx, beg, end))
            beg = end
        return out

    def _fwd_mm(a, Wt, cu, segs, width):
        """rows of a [M, K] times Wt[g] [K, width] per group -> [M, width] bf16."""
        if ffn["mode"] == "grouped":
            return _gmm(a, Wt, cu)
        out = torch.empty(a.shape[0], width, dtype=torch.bfloat16, device=a.device)
        for gidx, b, e in segs:
            torch.mm(a[b:e], Wt[gidx], out=out[b:e])
        return out

    def _bwd_mm(dy, Wt, cu, segs, width, accumulate_into=None):
        """dy [M, N] times Wt[g]^T per group -> [M, width] bf16 (optionally added to a previous result)."""
        if ffn["mode"] == "grouped":
            r = _gmm(dy, Wt.transpose(1, 2), cu)
            return r if accumulate_into is None else accumulate_into + r
        if accumulate_into is None:
            out = torch.empty(dy.shape[0], width, dtype=torch.bfloat16, device=dy.device)
            for gidx, b, e in segs:
                torch.mm(dy[b:e], Wt[gidx].t(), out=out[b:e])
            return out
        for gidx, b, e in segs:
            accumulate_into[b:e].addmm_(dy[b:e], Wt[gidx].t())
        return accumulate_into

    def _wgrad(a, dy, cu, segs, out):
        """out[g] = a_g^T dy_g in fp32, written in place; groups without rows: local ones get zeros."""
        if ffn["mode"] == "grouped":
            out.copy_(_gmm_wgrad(a, dy, cu, 2 * epn))
            return
        seen = set()
        for gidx, b, e in segs:
            torch.mm(a[b:e].t(), dy[b:e], out_dtype=torch.float32, out=out[gidx])
            seen.add(gidx)
        for gidx in range(epn):
            if gidx not in seen:
                out[gidx].zero_()

    class MoE(torch.autograd.Function):
        @staticmethod
        def forward(ctx, hidden, w_sk, topk, tpe):
            x, w_nvs, cu, plan = buffer.dispatch(hidden, w_sk, topk, tpe)
            buffer.prefetch_weight(plan=plan, **prefetch_kwargs())
            segs = _segments(cu) if ffn["mode"] == "loop" else None
            Wg, Wu, Wd = W["gate"][rank], W["up"][rank], W["down"][rank]
            gp, up = _fwd_mm(x, Wg, cu, segs, Hp), _fwd_mm(x, Wu, cu, segs, Hp)
            act = fused["fwd"](gp, up, w_nvs)
            y = _fwd_mm(act, Wd, cu, segs, H)
            out, _, _ = buffer.combine(plan=plan, hidden_nvsh=y)
            ctx.saved = (plan, cu, segs, x, w_nvs, act, gp, up)
            return out

        @staticmethod
        def backward(ctx, grad_out):
            plan, cu, segs, x, w_nvs, act, gp, up = ctx.saved
            Wg, Wu, Wd = W["gate"][rank], W["up"][rank], W["down"][rank]
            dy, _, _, _ = buffer.dispatch(grad_out.contiguous(), plan=plan)
            dA = _bwd_mm(dy, Wd, cu, segs, Hp)
            _wgrad(act, dy, cu, segs, Gd["down"][rank])
            dg, du, dw = fused["bwd"](dA, gp, up, w_nvs)
            dx = _bwd_mm(dg, Wg, cu, segs, H)
            dx = _bwd_mm(du, Wu, cu, segs, H, accumulate_into=dx)
            _wgrad(x, dg, cu, segs, Gd["gate"][rank])
            _wgrad(x, du, cu, segs, Gd["up"][rank])
            gh, gw, _ = buffer.combine(plan=plan, hidden_nvsh=dx, route_weights_nvs=dw.contiguous())
            if R > 1:
                buffer.reduce_grad(plan=plan, **reduce_kwargs())
            return gh, gw, None, None

    lr = 1e-3

    def step(x, before_optimizer=None):
        x.requires_grad_(True)
        w, topk, tpe = route(x)
        y = MoE.apply(x, w, topk, tpe)
        loss = mean_square(y)
        loss.backward()
        if before_optimizer is not None:
            before_optimizer()
        with torch.no_grad():
            for n in shapes:
                fused["sgd"](W[n][rank, :epn], Gd[n][rank, :epn], lr)
            router.add_(router.grad.to(router.dtype), alpha=-lr)
            router.grad = None
        x.grad = None
        return loss.detach()

    def sync():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def mx(v):
        if world == 1:
            return v
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    def maxvio_of(tpe):
        t = tpe.clone().double()
        if world > 1:
            dist.all_reduce(t)
        return float(t.max() / t.mean() - 1.0)

    def calibrate(x, target):
        def mv(scale):
            state["bias"] = bias_base * scale
            with torch.no_grad():
                return maxvio_of(route(x)[2])
        floor = mv(0.0)
        if target <= floor:
            state["bias"] = bias_base * 0.0
            return floor
        lo, hi, best = 1e-3, 50.0, (0.0, floor)
        for _ in range(40):
            mid = (lo * hi) ** 0.5
            v = mv(mid)
            if abs(v - target) < abs(best[1] - target):
                best = (mid, v)
            if abs(v - target) <= max(0.02 * target, 0.005):
                break
            lo, hi = (mid, hi) if v < target else (lo, mid)
        state["bias"] = bias_base * best[0]
        return best[1]

    gen = torch.Generator().manual_seed(100 + rank)
    host = [torch.randn(S, H, generator=gen).to(torch.bfloat16).pin_memory() for _ in range(2)]
    devb = [b.cuda() for b in host]
    realised = calibrate(devb[0], args.maxvio)
    W_ = max(3, args.warmup)
    # which form of the expert GEMMs is faster here: two untimed steps each (after one to warm up), max over ranks
    trial = {}
    forms = ["grouped", "loop"] if hasattr(torch, "_grouped_mm") and "MOONEP_REF_FFN" not in os.environ else [ffn["mode"]]
    if not hasattr(torch, "_grouped_mm"):
        forms = ["loop"]
    for mode in forms:
        ffn["mode"] = mode
        try:
            step(devb[0].detach())
            sync()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(2):
                step(devb[i % 2].detach())
            e1.record()
            sync()
            trial[mode] = mx(e0.elapsed_time(e1) / 2)
        except Exception:      # noqa: BLE001  (e.g. an fp32-output GEMM this build of the library lacks)
            trial[mode] = float("inf")
        ok = torch.tensor([0 if trial[mode] == float("inf") else 1], device=dev)
        if world > 1:
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok) == 0:
            trial[mode] = float("inf")
    ffn["mode"] = min(trial, key=trial.get)
    sampler = _clock_sampler(int(os.environ.get("LOCAL_RANK", "0")))     # started before the warm-up, as in the other arm
    for _ in range(W_):
        step(devb[0].detach())
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(devb[i % 2].detach())
    e1.record()
    sync()
    ms = mx(e0.elapsed_time(e1) / args.steps)
    clocks = sampler.stop() if sampler is not None else {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
    copy_stream = torch.cuda.Stream()

    def fetch(i, after=None):
        with torch.cuda.stream(copy_stream):
            if after is not None:
                copy_stream.wait_event(after)
            x = host[i % 2].to("cuda", non_blocking=True)
            ev = copy_stream.record_event()
        return x, ev

    # same protocol as the main arm: the batch of step i+1 is copied from pinned host memory while the
    # optimizer of step i runs (a host-to-device copy slows communication kernels it overlaps with; the
    # optimizer is local work), only the first batch is copied up front; the loss of step i goes to pinned
    # host memory asynchronously and is read after step i+1 has been queued (the last one after the loop)
    loss_host = [torch.zeros(1, dtype=torch.float32).pin_memory() for _ in range(2)]
    done = [None, None]
    lv = None

    def read_loss(i):
        done[i % 2].synchronize()
        return float(loss_host[i % 2][0])

    sync()
    t0 = time.perf_counter()
    nxt = [fetch(0)]
    for i in range(args.steps):
        x, ev = nxt[0]

        def stage(i=i):
            if i + 1 < args.steps:
                nxt[0] = fetch(i + 1, after=torch.cuda.current_stream().record_event())

        torch.cuda.current_stream().wait_event(ev)
        x.record_stream(torch.cuda.current_stream())
        loss_host[i % 2].copy_(step(x, stage).reshape(1).float(), non_blocking=True)
        done[i % 2] = torch.cuda.current_stream().record_event()
        if i > 0:
            lv = read_loss(i - 1)
    lv = read_loss(args.steps - 1)
    sync()
    e2e_ms = mx((time.perf_counter() - t0) * 1e3 / args.steps)
    def best_of(fn, n=5, reps=3):
        """Same protocol as the main arm: n back-to-back calls between CUDA events, max over ranks, best of
        ``reps`` batches (a pause of the host stretches the batch it falls into)."""
        best = float("inf")
        for _ in range(reps):
            sync()
            if world > 1:
                dist.barrier()
            e0.record()
            for _ in range(n):
                fn()
            e1.record()
            sync()
            best = min(best, mx(e0.elapsed_time(e1) / n * 1e3))
        return best

    def time_ops(fns, n=5):
        out = []
        for fn in fns:
            for _ in range(2):
                fn()
            out.append(round(best_of(fn, n), 1))
        return out

    def comm_times(xin, w, topk, tpe):
        """The four public collectives one by one (same calls and flags as the main arm)."""
        h, wn, cu, plan = buffer.dispatch(xin, w, topk, tpe, zero_copy=True, router_weights_zero_copy=True)
        ops = [lambda: buffer.dispatch(xin, w, topk, tpe, zero_copy=True, router_weights_zero_copy=True)]
        if world > 1:
            ops.append(lambda: buffer.prefetch_weight(plan=plan, **prefetch_kwargs()))
        ops.append(lambda: buffer.combine(plan=plan, hidden_nvsh=h, route_weights_nvs=wn, zero_copy=True,
                                          router_weights_zero_copy=True))
        if world > 1:
            ops.append(lambda: buffer.reduce_grad(plan=plan, **reduce_kwargs()))
        t = time_ops(ops)
        if world > 1:
            return {"dispatch_us": t[0], "prefetch_us": t[1], "combine_us": t[2], "reduce_grad_us": t[3]}
        return {"dispatch_us": t[0], "prefetch_us": None, "combine_us": t[1], "reduce_grad_us": None}

    sweep = []
    if not args.no_sweep:
        for mv in SWEEP:
            real = calibrate(devb[0], mv)
            step(devb[0].detach())
            sync()
            e0.record()
            for i in range(3):
                step(devb[i % 2].detach())
            e1.record()
            sync()
            sms = mx(e0.elapsed_time(e1) / 3)
            with torch.no_grad():
                w, topk, tpe = route(devb[0])

            def comm():
                h, wn, cu, plan = buffer.dispatch(devb[0], w, topk, tpe, zero_copy=True, router_weights_zero_copy=True)
                if world > 1:
                    buffer.prefetch_weight(plan=plan, **prefetch_kwargs())
                buffer.combine(plan=plan, hidden_nvsh=h, route_weights_nvs=wn, zero_copy=True, router_weights_zero_copy=True)

            for _ in range(3):
                comm()
            sweep.append({"maxvio_target": mv, "maxvio": round(real, 3), "step_ms": round(sms, 3),
                          "dispatch_combine_us": round(best_of(comm), 1),
                          **comm_times(devb[0], w, topk, tpe)})
    calibrate(devb[0], args.maxvio)
    with torch.no_grad():
        w_, topk_, tpe_ = route(devb[0])
    comm = comm_times(devb[0], w_, topk_, tpe_)
    comm["sequence_us"] = round(sum(v for v in comm.values() if v is not None), 1)
    tokens = S * world
    out = {"metric": "moe_layer_train_step_tokens_per_s", "value": tokens / (ms * 1e-3), "unit": "tokens/s",
           "n_gpus": world, "steps": args.steps, "warmup": W_, "ms_per_step": ms, "higher_is_better": True,
           "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "reference",
           "config": {"model": f"{args.model}-shape MoE layer (H={H}, H'={Hp}, K={K}, E={E}, epn={epn})",
                      "global_batch": tokens, "seq_len": S, "parallelism": f"ep{world}", "token_padding": 128,
                      "num_sms": 32, "maxvio_target": args.maxvio, "maxvio": round(realised, 3),
                      "l2": "inputs larger than L2 (multi-GB working set per step)"},
           "notes": {"step": "router + dispatch + grouped GEMM fwd/bwd + combine + reduce_grad + SGD",
                     "launch": "launched from Python", "path": "default",
                     "e2e_input_copy": "on a side stream, starting when the step before its use reaches the optimizer",
                     "dispatch": "the GEMMs start after the dispatch call returns",
                     "combine": "pulled from the peers' shards after the down GEMM",
                     "comm": "reference moonep.Buffer (unmodified)",
                     "expert_ffn": ("torch._grouped_mm" if ffn["mode"] == "grouped" else "one cuBLAS torch.mm per expert group")
                                   + f"; SwiGLU and SGD: {fused['how']}; trial step ms: {trial}"},
           "comm": comm,
           "clocks": {"sm_mhz": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"], "reasons": clocks["reasons"]},
           "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                   "h2d_bytes_per_step": S * H * 2, "d2h_bytes_per_step": 4},
           "loss": lv, "maxvio_sweep": sweep}
    if rank == 0:
        print(json.dumps(out), flush=True)
    buffer.destroy()
    dist.destroy_process_group()
