"""Dispatch with per-tile ready flags (``dispatch_ready``): same rows, weights and plans as the plain
dispatch, correct send list / source table / flag state, a GEMM that consumes the shard while the
dispatch kernel is still running, and the bounded wait of a consumer whose tile never completes."""
import numpy as np
import pytest
import torch

from moonep_b200 import engine
from moonep_b200.sim import plan_cluster, ops as simops
from moonep_b200.sim import flags as simflags
from moonep_b200.sim.local_cluster import LocalCluster

from gpu_helpers import make_topk, traceable_hidden, check_plans, defined_rows

pytestmark = pytest.mark.gpu

CASES = [
    # name            S    K  epn  H     R  sms pad  routing
    ("r1",            96,  4, 4,   256,  1, 2,  16,  "random"),
    ("r2_biased",     128, 4, 4,   512,  2, 2,  32,  "biased"),
    ("r4_pad128",     192, 8, 4,   256,  4, 3,  128, "biased"),
    ("r4_dup_heavy",  64,  8, 2,   1024, 4, 2,  16,  "random"),
    ("r8_k1",         80,  1, 3,   256,  8, 1,  16,  "random"),
    ("r3_deep_ring",  300, 6, 5,   64,   3, 2,  8,   "biased"),
    ("r8_k8",         96,  8, 2,   512,  8, 2,  16,  "biased"),
    ("r8_wide_rows",  64,  8, 4,   7168, 8, 1,  128, "random"),
]


def _setup(S, K, epn, H, R, sms, pad, kind, budget_ms=4000):
    E = R * epn
    topk, tpe = make_topk(kind, S, K, E, R, seed=11, sigma=1.5)
    cp = plan_cluster(np.stack([t.numpy() for t in topk]), E, pad)
    cl = LocalCluster(S, H, K, E, R, num_sms=sms, token_padding=pad, budget_ms=budget_ms)
    dev = cl.device
    hidden = [traceable_hidden(S, H, r) for r in range(R)]
    weights = [(torch.arange(S * K, dtype=torch.int32) + r * S * K + 1).view(torch.float32).reshape(S, K) for r in range(R)]
    return cl, cp, topk, tpe, hidden, weights, dev


def _poison(cl):
    for s in cl._states:
        s.hidden_local.view(torch.int16).fill_(0x5555)
        s.weights_local.view(torch.int32).fill_(0x55555555)


def _check_rows(cl, cp, hidden, weights, R):
    eh, ew = simops.dispatch(cp, [h.view(torch.int16).float() for h in hidden],
                             [w.view(torch.int32).float() for w in weights], fill=-1.0)
    for d in range(R):
        m = defined_rows(cp, d)
        got = cl._states[d].hidden_local.cpu().view(torch.int16).float()
        assert torch.equal(got[m], eh[d][m]), f"rank {d}: dispatched rows differ"
        gw = cl._states[d].weights_local.cpu().view(torch.int32).float()
        assert torch.equal(gw[m], ew[d][m]), f"rank {d}: dispatched weights differ"


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_flagged_dispatch_rows_tables_and_flags(case, cuda_device):
    _, S, K, epn, H, R, sms, pad, kind = case
    cl, cp, topk, tpe, hidden, weights, dev = _setup(S, K, epn, H, R, sms, pad, kind)
    g = cl.geo
    _poison(cl)
    hd, wd = [h.to(dev) for h in hidden], [w.to(dev) for w in weights]
    oh, ow, cus, plans, ev = cl.dispatch_ready(hd, wd, [t.to(dev) for t in topk], [t.to(dev) for t in tpe])
    torch.cuda.synchronize()
    cl.check()
    check_plans(plans, cus, cp, R)
    _check_rows(cl, cp, hidden, weights, R)
    want_src = simflags.rowsrc_tables(cp)
    for r in range(R):
        st = cl._states[r]
        # send list: the right entries, bucket by bucket in ascending bucket order
        ents, buckets = simflags.wire_entries(cp, r)
        n = int(plans[r].send_meta[0])
        assert n == len(ents) and int(plans[r].send_meta[1]) == int(cp.cu_seqlens[r, -1])
        got = plans[r].send_list[:n].cpu().numpy()
        bucket_of = dict(zip(ents.tolist(), buckets.tolist()))
        assert sorted(got.tolist()) == sorted(ents.tolist()), f"rank {r}: send list names other entries"
        gb = np.asarray([bucket_of[e] for e in got.tolist()])
        assert np.all(np.diff(gb) >= 0), f"rank {r}: send list is not ordered by (tile, destination)"
        # source table of every slot the dispatch defines
        rs = cl.heap.view(r, g.off_rowsrc, (g.NvS,), torch.int32).cpu().numpy()
        m = want_src[r] != -2
        assert np.array_equal(rs[m], want_src[r][m]), f"rank {r}: rowsrc differs"
        # flags: one arrival per slot, every used tile complete at epoch 1
        ready = cl.heap.view(r, g.off_ready, (g.ntiles,), torch.int32).cpu().numpy()
        rows = np.minimum(128, g.NvS - 128 * np.arange(g.ntiles))
        assert np.array_equal(ready, rows), f"rank {r}: arrival counters {ready} != {rows}"
        used = (int(cp.cu_seqlens[r, -1]) + 127) // 128
        done = st.scratch["tile_done"].cpu().numpy()
        assert np.all(done[:used] == 1) and np.all(done[used:] == 0)
        assert int(st.scratch["flag_epoch"][0]) == 1

    # the plan drives a second, hidden-only dispatch (backward of combine): other payload, epoch 2
    hidden2 = [traceable_hidden(S, H, r + 5) for r in range(R)]
    _poison(cl)
    cl.dispatch_ready([h.to(dev) for h in hidden2], None, plans=plans)
    torch.cuda.synchronize()
    cl.check()
    eh, _ = simops.dispatch(cp, [h.view(torch.int16).float() for h in hidden2], None, fill=-1.0)
    for d in range(R):
        m = defined_rows(cp, d)
        assert torch.equal(cl._states[d].hidden_local.cpu().view(torch.int16).float()[m], eh[d][m])
        ready = cl.heap.view(d, g.off_ready, (g.ntiles,), torch.int32).cpu().numpy()
        assert np.array_equal(ready, 2 * np.minimum(128, g.NvS - 128 * np.arange(g.ntiles)))
    # and the plain dispatch still works on the same Buffer with the same plan
    _poison(cl)
    cl.dispatch(hd, wd, plans=plans)
    torch.cuda.synchronize()
    cl.check()
    _check_rows(cl, cp, hidden, weights, R)
    c = engine.read_counters(cl._states[0])
    assert c["dispatches"] == 3 and c["rows_sent"] > 0 and sum(c["rows_sent_to"]) == c["rows_sent"]


@pytest.mark.parametrize("R,mode", [(1, "gate_up"), (2, "gate_up"), (4, "gate_up"), (2, "dgrad")])
def test_gemm_consumes_tiles_while_dispatch_runs(R, mode, cuda_device):
    """The GEMM is launched on the main stream while the flagged dispatch runs on another stream; it
    may only load a tile once its flag is up, so its result must equal the GEMM on the complete shard
    (a tile loaded early would contain the poison pattern)."""
    from moonep_b200.ops import grouped_gemm as gg
    S, K, epn, H, Hp, pad, sms = 256, 4, 5, 256, 256, 128, 2
    cl, cp, topk, tpe, hidden, weights, dev = _setup(S, K, epn, H, R, sms, pad, "biased")
    g = cl.geo
    gen = torch.Generator(device="cuda").manual_seed(3)
    hid = [(torch.randn(S, H, device=dev, generator=gen) * 0.5).to(torch.bfloat16) for _ in range(R)]
    wts = [torch.rand(S, K, device=dev, generator=gen) for _ in range(R)]
    G = 2 * epn
    Wg = [(torch.randn(G, H, Hp, device=dev, generator=gen) * 0.05).to(torch.bfloat16) for _ in range(R)]
    Wu = [(torch.randn(G, H, Hp, device=dev, generator=gen) * 0.05).to(torch.bfloat16) for _ in range(R)]
    for rep in range(2):            # second round: epoch 2 on the same flags
        for s in cl._states:
            s.hidden_local.fill_(float("nan"))
        torch.cuda.synchronize()
        oh, ow, cus, plans, ev = cl.dispatch_ready(hid, wts, [t.to(dev) for t in topk], [t.to(dev) for t in tpe])
        outs = []
        for r in range(R):
            ready = cl.tile_ready(r)
            x, w = cl._states[r].hidden_local, cl._states[r].weights_local
            if mode == "gate_up":
                act = torch.zeros(g.NvS, Hp, dtype=torch.bfloat16, device=dev)
                gg.gate_up(x, Wg[r], Wu[r], cus[r], act, None, row_scale=w, num_ctas=min(16, ready.free_sms), ready=ready)
            else:
                act = torch.zeros(g.NvS, H, dtype=torch.bfloat16, device=dev)
                gg.dgrad(x, Wg[r].transpose(1, 2).contiguous(), cus[r], act, num_ctas=min(16, ready.free_sms), ready=ready)
            outs.append(act)
        torch.cuda.synchronize()
        cl.check()
        gg.check_status()
        for r in range(R):
            x = cl._states[r].hidden_local.float()
            w = cl._states[r].weights_local
            cu = cus[r].cpu().tolist()
            ref = torch.zeros_like(outs[r], dtype=torch.float32)
            beg = 0
            for gi, end in enumerate(cu):
                if end > beg:
                    xs = x[beg:end]
                    if mode == "gate_up":
                        ref[beg:end] = torch.nn.functional.silu(xs @ Wg[r][gi].float()) * (xs @ Wu[r][gi].float()) * w[beg:end, None]
                    else:
                        ref[beg:end] = xs @ Wg[r][gi].float()
                beg = end
            m = defined_rows(cp, r).to(dev)
            assert torch.isfinite(outs[r].float()[m]).all(), f"rank {r}: a tile was loaded before it was complete"
            err = (outs[r].float()[m] - ref[m]).norm() / (ref[m].norm() + 1e-12)
            assert float(err) < 2e-2, f"rank {r} round {rep}: {float(err)}"


def test_consumer_wait_runs_out_when_no_dispatch_completes_the_tile(cuda_device):
    """A flag epoch is opened but no dispatch is launched: the tile can never complete. The waits give
    up after the budget and report it; nothing traps and the context stays usable."""
    from moonep_b200.ops import grouped_gemm as gg
    S, K, epn, H, Hp, pad = 128, 2, 2, 256, 256, 128
    cl = LocalCluster(S, H, K, epn, 1, num_sms=2, token_padding=pad, budget_ms=30)
    st = cl._states[0]
    engine.launch_flag_epoch_bump(cl._states)
    engine.launch_tile_wait_probe(st, 0)
    torch.cuda.synchronize()
    assert engine.failed(st)                   # the host-visible copy is already set
    with pytest.raises(engine.MoonEPTimeout) as ei:
        cl.check()
    assert ei.value.status["code"] == 4 and ei.value.status["kernel"] == 10
    # the GEMM's producer gives up in the same way (its own budget comes from the environment)
    import os
    old = os.environ.get("MOONEP_WAIT_BUDGET_MS")
    os.environ["MOONEP_WAIT_BUDGET_MS"] = "30"
    try:
        g = cl.geo
        x = st.hidden_local
        cu = torch.tensor([128, 256, 256, 256], dtype=torch.int32, device="cuda")
        Wg = torch.zeros(4, H, Hp, dtype=torch.bfloat16, device="cuda")
        act = torch.zeros(g.NvS, Hp, dtype=torch.bfloat16, device="cuda")
        gg.gate_up(x, Wg, Wg, cu, act, None, num_ctas=4, ready=cl.tile_ready(0))
        torch.cuda.synchronize()
        assert gg.failed("cuda")
        with pytest.raises(RuntimeError, match="grouped GEMM aborted: code 4"):
            gg.check_status()
        assert not gg.failed("cuda")
    finally:
        if old is None:
            os.environ.pop("MOONEP_WAIT_BUDGET_MS")
        else:
            os.environ["MOONEP_WAIT_BUDGET_MS"] = old
    y = torch.ones(4, device="cuda") * 2
    assert float(y.sum()) == 8.0


@pytest.mark.parametrize("R,epn", [(4, 4), (2, 5)])
def test_prefetch_raises_one_flag_per_landed_slot(R, epn, cuda_device):
    """Every slot that received an expert carries the launch's prefetch epoch afterwards, every other
    slot's flag is untouched; the next launch stamps the next epoch (the per-slot chunk counters reset
    themselves)."""
    from gpu_helpers import run_case
    S, K, H = 200, 6, 64
    cl, cp, plans, *_ = run_case(S, K, epn, H, R, 3, 16, "biased", sigma=2.0, with_weights=False)
    assert (cp.experts_to_copy >= 0).any(), "case must produce redundant experts"
    dev, g = cl.device, cl.geo
    rows, cols = 72, 40                 # 5760 B per expert and tensor: several 64 KB chunks only with all three
    gen = torch.Generator().manual_seed(5)
    names = ("gate", "up", "down")
    local = {n: [torch.randn(epn, rows * 9, cols, generator=gen).to(torch.bfloat16) for _ in range(R)] for n in names}
    pools = {n: cl.make_pool((epn, rows * 9, cols), torch.bfloat16, 0)[0] for n in names}
    pairs = [[(local[n][r].to(dev), pools[n]) for n in names] for r in range(R)]
    for epoch in (1, 2):
        cl.prefetch(plans, pairs)
        torch.cuda.synchronize()
        cl.check()
        for r in range(R):
            flags = cl.heap.view(r, g.off_slotflag, (g.epn,), torch.int32).cpu().numpy()
            want = np.where(cp.experts_to_copy[r] >= 0, epoch, 0)
            assert np.array_equal(flags, want), f"rank {r}: slot flags {flags} != {want}"
            assert int(cl._states[r].scratch["slot_done"].abs().sum()) == 0, "chunk counters did not reset"
            assert int(cl._states[r].scratch["pf_epoch"][0]) == epoch


def test_gemm_waits_for_prefetch_slots(cuda_device):
    """gate/up over ``[local | slots]`` with slot flags: groups of prefetched experts are computed once
    their flag is up (result equals the unflagged GEMM); when a slot never lands the wait gives up."""
    import os
    from moonep_b200.ops import grouped_gemm as gg
    S, K, epn, H, Hp, pad = 128, 2, 2, 256, 256, 128
    cl = LocalCluster(S, H, K, epn, 1, num_sms=2, token_padding=pad, budget_ms=30)
    st, g = cl._states[0], cl.geo
    gen = torch.Generator(device="cuda").manual_seed(1)
    x = (torch.randn(512, H, device="cuda", generator=gen) * 0.5).to(torch.bfloat16)
    cu = torch.tensor([128, 256, 384, 512], dtype=torch.int32, device="cuda")      # groups 2, 3 = slots 0, 1
    W = (torch.randn(4, H, Hp, device="cuda", generator=gen) * 0.05).to(torch.bfloat16)
    ref = torch.zeros(512, Hp, dtype=torch.bfloat16, device="cuda")
    gg.gate_up(x, W, W, cu, ref, None)
    slots = cl.slot_ready(0)
    flags = cl.heap.view(0, g.off_slotflag, (g.epn,), torch.int32)
    st.scratch["pf_epoch"][0] = 3
    flags.fill_(3)                      # both slots landed in prefetch epoch 3
    out = torch.zeros_like(ref)
    gg.gate_up(x, W, W, cu, out, None, slots=slots)
    torch.cuda.synchronize()
    gg.check_status()
    assert torch.equal(out, ref)
    flags[1] = 2                        # slot 1 still holds the previous launch's expert
    old = os.environ.get("MOONEP_WAIT_BUDGET_MS")
    os.environ["MOONEP_WAIT_BUDGET_MS"] = "30"
    try:
        gg.gate_up(x, W, W, cu, out, None, slots=slots)
        torch.cuda.synchronize()
        with pytest.raises(RuntimeError, match="grouped GEMM aborted: code 4"):
            gg.check_status()
    finally:
        if old is None:
            os.environ.pop("MOONEP_WAIT_BUDGET_MS")
        else:
            os.environ["MOONEP_WAIT_BUDGET_MS"] = old


def test_a_failed_wait_stops_the_next_public_call(cuda_device, monkeypatch):
    """Once a kernel of a Buffer has given up a wait, the next public op raises at its entry (the
    failure code is mirrored into host memory, so no synchronisation is needed to notice), instead of
    launching more work on unsynchronised data; ``reset()`` makes the Buffer usable again."""
    from moonep_b200 import Buffer
    monkeypatch.setenv("MOONEP_WAIT_BUDGET_MS", "30")
    S, H, K, E = 64, 256, 2, 4
    buf = Buffer(S, H, K, E, 1, num_sms=2, token_padding=16)
    x = torch.randn(S, H, device="cuda").to(torch.bfloat16)
    topk = torch.randint(0, E, (S, K), dtype=torch.int32, device="cuda")
    tpe = torch.bincount(topk.flatten().long(), minlength=E).to(torch.int32)
    w = torch.rand(S, K, device="cuda")
    buf.dispatch(x, w, topk, tpe)
    assert buf.healthy()
    st = buf._states[0]
    engine.launch_flag_epoch_bump([st])
    engine.launch_tile_wait_probe(st, 0)          # nothing completes this tile: the wait runs out
    torch.cuda.synchronize()
    assert not buf.healthy()
    with pytest.raises(engine.MoonEPTimeout):
        buf.dispatch(x, w, topk, tpe)
    with pytest.raises(engine.MoonEPTimeout):
        buf.combine(plan=None, hidden_nvsh=None)
    buf.reset()
    assert buf.healthy()
    h, wn, cu, plan = buf.dispatch(x, w, topk, tpe)
    torch.cuda.synchronize()
    buf.check()
    buf.destroy()
