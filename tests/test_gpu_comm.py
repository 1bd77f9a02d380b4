"""GPU tests of planning / dispatch / combine / prefetch / reduce_grad against the CPU oracle.
All R ranks run on one GPU through LocalCluster (one cooperative launch hosts every rank)."""
import numpy as np
import pytest
import torch

from moonep_b200.sim import ops as simops

pytestmark = pytest.mark.gpu

from gpu_helpers import run_case, defined_rows  # noqa: E402

CASES = [
    # name, S, K, epn, H, R, num_sms, pad, routing
    ("tiny_r1", 1, 1, 1, 64, 1, 1, 1, "random"),
    ("r1_balanced", 128, 4, 4, 256, 1, 4, 16, "balanced"),
    ("r2_random", 96, 4, 3, 128, 2, 3, 8, "random"),
    ("r2_all_remote", 64, 2, 2, 128, 2, 2, 16, "all_remote"),
    ("r4_single_expert", 40, 3, 2, 64, 4, 2, 8, "single_expert"),
    ("r4_duplicate_topk", 33, 4, 3, 64, 4, 2, 4, "duplicate_topk"),
    ("r4_all_local", 50, 4, 4, 64, 4, 3, 128, "all_local"),
    ("r8_balanced", 256, 8, 8, 256, 8, 4, 128, "balanced"),
    ("r8_biased", 256, 8, 8, 512, 8, 4, 128, "biased"),
    ("r8_heavy", 300, 6, 5, 128, 8, 3, 32, "biased"),
    ("r8_k32", 64, 32, 8, 64, 8, 2, 16, "random"),
    ("r3_odd", 77, 5, 7, 72, 3, 5, 5, "random"),
    ("r2_multi_vblock", 700, 8, 16, 64, 2, 2, 64, "biased"),
]


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_dispatch_combine(case, cuda_device):
    _, S, K, epn, H, R, num_sms, pad, kind = case
    sigma = 5.0 if case[0] == "r8_heavy" else 1.0
    cl, cp, plans, cus, hidden, weights, topk, tpe, oh, ow = run_case(S, K, epn, H, R, num_sms, pad, kind, sigma=sigma)
    dev = cuda_device
    # combine of small-integer payloads is exact: use value = (slot index mod 7) + 1 per row
    ys = []
    for d in range(R):
        y = torch.zeros(cp.NvS, H, dtype=torch.bfloat16)
        y[:] = ((torch.arange(cp.NvS) % 7) + 1)[:, None].to(torch.bfloat16)
        ys.append(y)
    outs, outw = cl.combine(plans, [y.to(dev) for y in ys], [w.to(dev) for w in ow])
    torch.cuda.synchronize()
    cl.check()
    eo, ewk = simops.combine(cp, [y.float() for y in ys], [w.cpu().view(torch.int32).float() for w in ow])
    for r in range(R):
        assert torch.equal(outs[r].cpu().float(), eo[r].to(torch.bfloat16).float()), f"rank {r}: combine mismatch"
        assert torch.equal(outw[r].cpu().view(torch.int32).float(), ewk[r]), f"rank {r}: gathered weights mismatch"
        assert torch.equal(outw[r].cpu().view(torch.int32), weights[r].view(torch.int32)), "weights must round-trip bit-exactly"


from shape_cases import case_params, case_id  # noqa: E402


@pytest.mark.parametrize("p", case_params(), ids=case_id)
def test_shape_list_plan_and_dispatch(p, cuda_device):
    """Planner outputs (bit-exact against the oracle, duplicate tables as sets), dispatched rows,
    route weights and zero-filled padding for every shape of the shared list, at every group
    size the shape allows; both planner kernels are reached (small and large expert counts)."""
    c, R = p
    num_sms = 1 if c.S * c.K < 64 else (4 if R > 2 else 6)
    cl, cp, plans, *_ = run_case(c.S, c.K, c.epn, c.H, R, num_sms, c.pad, c.routing, seed=c.seed, sigma=c.sigma)
    for r in range(R):
        assert int(plans[r].remote_stats[0]) == int((cp.experts_to_copy[r] >= 0).sum())
    cl.heap.close()


def test_combine_rounding(cuda_device):
    """randn payloads: duplicates rounded once locally, then one final rounding (<= 1 bf16 ulp)."""
    S, K, epn, H, R = 128, 8, 4, 256, 4
    cl, cp, plans, cus, hidden, weights, topk, tpe, oh, ow = run_case(S, K, epn, H, R, 4, 32, "biased")
    g = torch.Generator().manual_seed(3)
    ys = [torch.randn(cp.NvS, H, generator=g).to(torch.bfloat16) for _ in range(R)]
    outs, _ = cl.combine(plans, [y.to(cuda_device) for y in ys])
    torch.cuda.synchronize()
    eo, _ = simops.combine(cp, ys)
    for r in range(R):
        assert torch.equal(outs[r].cpu(), eo[r]), f"rank {r}: combine differs from the emulated rounding order"


def test_plan_reuse_and_repeat(cuda_device):
    """Backward path: dispatch with a saved plan (no planning, plan untouched), many times."""
    S, K, epn, H, R = 96, 4, 4, 128, 4
    cl, cp, plans, cus, hidden, weights, topk, tpe, oh, ow = run_case(S, K, epn, H, R, 3, 16, "biased")
    snap = [p.clone() for p in plans]
    ref = [h.clone() for h in oh]
    dev = cuda_device
    for it in range(5):
        for s in cl._states:
            s.hidden_local.view(torch.int16).fill_(0x3333)
        oh2, ow2, cu2, plans2 = cl.dispatch([h.to(dev) for h in hidden], None, plans=snap)
        torch.cuda.synchronize()
        cl.check()
        assert all(c is None for c in cu2) and all(w is None for w in ow2)
        assert all(a is b for a, b in zip(plans2, snap))
        for d in range(R):
            m = defined_rows(cp, d)
            assert torch.equal(oh2[d].cpu().view(torch.int16)[m], ref[d].cpu().view(torch.int16)[m])
            for name in ("dst", "dup_groups", "dup_loffs", "dup_counts", "experts_to_copy"):
                assert torch.equal(getattr(snap[d], name), getattr(plans[d], name))
    # fresh dispatches back to back (barrier epochs keep advancing)
    for it in range(3):
        cl.dispatch([h.to(dev) for h in hidden], None, [t.to(dev) for t in topk], [t.to(dev) for t in tpe])
    torch.cuda.synchronize()
    cl.check()


@pytest.mark.parametrize("R,epn,pad_elems", [(4, 4, 0), (8, 3, 24), (2, 5, 8)])
def test_prefetch_and_reduce(R, epn, pad_elems, cuda_device):
    S, K, H = 200, 6, 64
    cl, cp, plans, *_ = run_case(S, K, epn, H, R, 3, 16, "biased", sigma=2.0, with_weights=False)
    assert (cp.experts_to_copy >= 0).any(), "case must produce redundant experts"
    dev = cuda_device
    rows, cols = 40, 24          # expert payload 40*24*2 B = 1920 B (multiple of 16, not of the chunk)
    g = torch.Generator().manual_seed(5)
    names = ("gate", "up", "down")
    local = {n: [torch.randn(epn, rows, cols, generator=g).to(torch.bfloat16) for _ in range(R)] for n in names}
    pools, flats = {}, {}
    for n in names:
        pools[n], flats[n] = cl.make_pool((epn, rows, cols), torch.bfloat16, pad_elems)
        flats[n].fill_(-123.0)
    pairs = [[(local[n][r].to(dev), pools[n]) for n in names] for r in range(R)]
    cl.prefetch(plans, pairs)
    torch.cuda.synchronize()
    cl.check()
    for n in names:
        exp = [torch.full((epn, rows, cols), -123.0, dtype=torch.bfloat16) for _ in range(R)]
        simops.prefetch(cp, local[n], exp)
        for r in range(R):
            assert torch.equal(pools[n][r].cpu(), exp[r]), f"{n}: prefetch slots of rank {r} differ"
        if pad_elems:
            per = epn * rows * cols
            gaps = flats[n].cpu().view(R, per + pad_elems)[:, per:]
            assert (gaps == -123.0).all(), "padding between ranks was overwritten"

    # --- reduce_grad (fp32, bitwise: fixed summation order)
    lg = {n: [torch.randn(epn, rows, cols, generator=g) for _ in range(R)] for n in names}
    rb = {n: [torch.randn(epn, rows, cols, generator=g) for _ in range(R)] for n in names}
    rpools, rflats, lgd = {}, {}, {}
    for n in names:
        rpools[n], rflats[n] = cl.make_pool((epn, rows, cols), torch.float32, pad_elems)
        rflats[n].fill_(-7.0)
        for r in range(R):
            rpools[n][r].copy_(rb[n][r])
        lgd[n] = [x.to(dev) for x in lg[n]]
    pairs = [[(lgd[n][r], rpools[n]) for n in names] for r in range(R)]
    cl.reduce_grad(plans, pairs)
    torch.cuda.synchronize()
    cl.check()
    for n in names:
        el = [x.clone() for x in lg[n]]
        er = [x.clone() for x in rb[n]]
        simops.reduce_grad(cp, el, er)
        for r in range(R):
            assert torch.equal(lgd[n][r].cpu(), el[r]), f"{n}: reduced grad of rank {r} differs (must be bitwise)"
            assert torch.equal(rpools[n][r].cpu(), er[r]), f"{n}: reduce slots of rank {r} differ"
    # second launch on the same cluster: barrier state must have reset itself
    cl.reduce_grad(plans, pairs)
    torch.cuda.synchronize()
    cl.check()


def test_bounded_wait_reports_timeout(cuda_device):
    """A wait on a flag nobody sets must give up after the budget and leave the context usable."""
    from moonep_b200 import engine
    from moonep_b200.sim.local_cluster import LocalCluster
    cl = LocalCluster(8, 64, 2, 4, 1, num_sms=1, token_padding=4, budget_ms=20.0)
    flag = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    engine.launch_wait_probe(cl._states[0], flag, 1)
    torch.cuda.synchronize()
    with pytest.raises(engine.MoonEPTimeout) as ei:
        cl.check()
    assert ei.value.status["code"] == 4 and ei.value.status["expected"] == 1
    # the context is still healthy
    assert float((torch.ones(4, device=cuda_device) * 2).sum()) == 8.0


def test_public_buffer_r1(cuda_device):
    """Public API on one rank: sync vs async, zero-copy aliasing, plan reuse."""
    from moonep_b200 import Buffer, MoonEPCommPlan
    S, H, K, E = 64, 128, 4, 8
    buf = Buffer(S, H, K, E, 1, num_sms=4, token_padding=16)
    g = torch.Generator(device="cuda").manual_seed(0)
    hidden = torch.randn(S, H, dtype=torch.bfloat16, device="cuda", generator=g)
    w = torch.rand(S, K, device="cuda", generator=g)
    topk = torch.randint(0, E, (S, K), dtype=torch.int32, device="cuda", generator=g)
    tpe = torch.bincount(topk.flatten(), minlength=E).to(torch.int32)
    h1, w1, cu1, plan1 = buf.dispatch(hidden, w, topk, tpe)
    buf.verify_plan(plan1)            # replicated planners agree; every rank receives S*K rows
    assert isinstance(plan1, MoonEPCommPlan) and tuple(h1.shape) == (buf.NvS, H)
    h2, w2, cu2, plan2, ev = buf.dispatch(hidden, w, topk, tpe, async_finish=True)
    ev.wait(torch.cuda.current_stream())
    torch.cuda.synchronize()
    n = int(cu1[-1])
    assert torch.equal(h1[:n], h2[:n]) and torch.equal(w1[:n], w2[:n]) and torch.equal(cu1, cu2)
    assert torch.equal(plan1.dst, plan2.dst)
    out, wsk, _ = buf.combine(plan=plan1, hidden_nvsh=h1, route_weights_nvs=w1)
    torch.cuda.synchronize()
    assert torch.equal(wsk, w)
    ref = (hidden.float() * K)       # each of the K copies comes back unweighted
    assert torch.allclose(out.float(), ref, rtol=2e-2, atol=2e-2)
    hz, wz, _, planz = buf.dispatch(hidden, w, topk, tpe, zero_copy=True, router_weights_zero_copy=True)
    assert hz.data_ptr() == buf.hidden_nvsh_buffer_view.data_ptr()
    outz, wz2, _ = buf.combine(plan=planz, hidden_nvsh=hz, route_weights_nvs=wz, zero_copy=True, router_weights_zero_copy=True)
    torch.cuda.synchronize()
    assert torch.equal(outz, out)
    with pytest.raises(AssertionError, match="alias"):
        buf.combine(plan=planz, hidden_nvsh=h1, zero_copy=True)
    hr, wr, cur, pr = buf.dispatch(hidden, plan=plan1)
    assert wr is None and cur is None and pr is plan1
    torch.cuda.synchronize()
    assert torch.equal(hr[:n], h1[:n])
    buf.check()
    buf.destroy()
    assert buf.destroyed
    buf.destroy()


def test_prefetch_with_scales_and_int8(cuda_device):
    """Six tensors in one launch: uint8 packed weights plus their block scales (byte-typed copy)."""
    R, epn, S, K, H = 4, 3, 150, 6, 64
    cl, cp, plans, *_ = run_case(S, K, epn, H, R, 3, 16, "biased", sigma=2.0, with_weights=False)
    assert (cp.experts_to_copy >= 0).any()
    dev = cuda_device
    g = torch.Generator().manual_seed(9)
    shapes = [((48, 32), torch.uint8), ((48, 32), torch.uint8), ((32, 48), torch.int8),
              ((48, 2), torch.uint8), ((48, 2), torch.uint8), ((32, 4), torch.uint8)]
    local, pools = [], []
    for shp, dt in shapes:
        local.append([torch.randint(0, 100, (epn, *shp), generator=g).to(dt) for _ in range(R)])
        pool, flat = cl.make_pool((epn, *shp), dt, pad_elems=16)
        flat.fill_(7)
        pools.append(pool)
    pairs = [[(local[i][r].to(dev), pools[i]) for i in range(6)] for r in range(R)]
    cl.prefetch(plans, pairs)
    torch.cuda.synchronize()
    cl.check()
    for i, (shp, dt) in enumerate(shapes):
        exp = [torch.full((epn, *shp), 7, dtype=dt) for _ in range(R)]
        simops.prefetch(cp, local[i], exp)
        for r in range(R):
            assert torch.equal(pools[i][r].cpu(), exp[r]), f"tensor {i}: slots of rank {r} differ"


def test_planner_large_expert_count(cuda_device):
    """E above the shared-memory table capacity takes the global-memory code paths."""
    from moonep_b200 import engine
    from moonep_b200.sim import plan_cluster
    from moonep_b200.sim.local_cluster import LocalCluster
    import numpy as np
    R, epn, S, K, pad = 2, 4200, 300, 4, 2
    E = R * epn
    g = torch.Generator().manual_seed(4)
    topk = [torch.randint(0, E, (S, K), dtype=torch.int32, generator=g) for _ in range(R)]
    for t in topk:                       # a few hot experts so that rank 1 needs help
        t[:, 0] = epn + (t[:, 0] % 3)
    tpe = [torch.bincount(t.flatten().long(), minlength=E).to(torch.int32) for t in topk]
    cp = plan_cluster(np.stack([t.numpy() for t in topk]), E, pad)
    cl = LocalCluster(S, 64, K, E, R, num_sms=2, token_padding=pad)
    st = cl._states
    plans, cus = zip(*[engine.allocate_plan(s) for s in st])
    engine.launch_planning(st, [t.reshape(-1).to(cuda_device) for t in topk], [t.to(cuda_device) for t in tpe], list(plans), list(cus))
    torch.cuda.synchronize()
    cl.check()
    for r in range(R):
        assert torch.equal(plans[r].dst.cpu().long(), torch.from_numpy(cp.dst[r]))
        assert torch.equal(cus[r].cpu().long(), torch.from_numpy(cp.cu_seqlens[r]))
        assert torch.equal(plans[r].experts_to_copy.cpu().long(), torch.from_numpy(cp.experts_to_copy))


def test_trace_stats_and_reset(cuda_device, monkeypatch):
    """Device timestamp ring, plan statistics and the collective reset of barrier state."""
    from moonep_b200 import Buffer, engine
    monkeypatch.setenv("MOONEP_TRACE", "1")
    S, H, K, E = 64, 128, 4, 8
    buf = Buffer(S, H, K, E, 1, num_sms=2, token_padding=16)
    g = torch.Generator(device="cuda").manual_seed(0)
    hidden = torch.randn(S, H, dtype=torch.bfloat16, device="cuda", generator=g)
    w = torch.rand(S, K, device="cuda", generator=g)
    topk = torch.randint(0, E, (S, K), dtype=torch.int32, device="cuda", generator=g)
    tpe = torch.bincount(topk.flatten(), minlength=E).to(torch.int32)
    h, wn, cu, plan = buf.dispatch(hidden, w, topk, tpe)
    buf.combine(plan=plan, hidden_nvsh=h)
    tr = engine.read_trace(buf._states[0])
    kernels = {k for _, k, _, _, _ in tr}
    assert 3 in kernels and 6 in kernels, "dispatch and combine must have left timestamps"
    assert all(a[0] <= b[0] for a, b in zip(tr, tr[1:]))
    st = buf.stats(plan)
    assert st["experts_received"] == 0 and st["dup_rows"] == int(plan.dup_counts[1]) and 0 <= st["dedup_ratio"] < 1
    buf.reset()
    h2, _, cu2, plan2 = buf.dispatch(hidden, w, topk, tpe)
    torch.cuda.synchronize()
    n = int(cu[-1])
    assert torch.equal(h2[:n], h[:n]) and torch.equal(cu2, cu) and torch.equal(plan2.dst, plan.dst)
    buf.check()
    buf.destroy()


def test_bad_inputs_raise(cuda_device):
    """Argument validation of the public API (messages a user can act on)."""
    from moonep_b200 import Buffer
    S, H, K, E = 32, 64, 2, 4
    buf = Buffer(S, H, K, E, 1, num_sms=1, token_padding=8)
    hidden = torch.zeros(S, H, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(S, K, device="cuda")
    topk = torch.zeros(S, K, dtype=torch.int32, device="cuda")
    tpe = torch.tensor([S * K, 0, 0, 0], dtype=torch.int32, device="cuda")
    with pytest.raises(AssertionError, match="topk_experts_sk and tokens_per_expert"):
        buf.dispatch(hidden, w)
    with pytest.raises(AssertionError, match="bf16"):
        buf.dispatch(hidden.float(), w, topk, tpe)
    with pytest.raises(AssertionError, match="int32"):
        buf.dispatch(hidden, w, topk.long(), tpe)
    with pytest.raises(AssertionError, match=r"\[E\] int32"):
        buf.dispatch(hidden, w, topk, tpe[:3])
    h, wn, cu, plan = buf.dispatch(hidden, w, topk, tpe)
    with pytest.raises(AssertionError, match="plan is required"):
        buf.combine(hidden_nvsh=h)
    with pytest.raises(AssertionError, match="NvS"):
        buf.combine(plan=plan, hidden_nvsh=h[:-1].contiguous())
    with pytest.raises(AssertionError, match="provided together"):
        buf.prefetch_weight(plan=plan, local_gate_weight=torch.zeros(4, 8, 8, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(AssertionError, match="provided together"):
        buf.reduce_grad(plan=plan, local_gate_grad=torch.zeros(4, 8, 8, device="cuda"))
    other = Buffer(S, H, K + 1, E, 1, num_sms=1, token_padding=8)
    with pytest.raises(AssertionError, match="another Buffer geometry"):
        other.dispatch(hidden, plan=plan)
    other.destroy()
    buf.destroy()
    with pytest.raises(AssertionError, match="destroyed"):
        buf.dispatch(hidden, w, topk, tpe)


def test_prefetch_and_reduce_beyond_2gib_offsets(cuda_device):
    """Expert payloads whose byte offsets inside a rank's pool exceed 2^31 (64-bit addressing)."""
    R, epn, S, K, H = 2, 3, 120, 4, 64
    cl, cp, plans, *_ = run_case(S, K, epn, H, R, 4, 8, "all_remote", with_weights=False)
    # force redundancy-free plan to still exercise slots: build a plan table by hand
    etc = torch.full((R, epn), -1, dtype=torch.int32)
    etc[0, 2] = 1 * epn + 2        # rank 0 slot 2 <- rank 1's last expert (offset > 2^31 in both pools)
    etc[1, 1] = 0 * epn + 2        # rank 1 slot 1 <- rank 0's last expert
    fake = [type(p)(**{**{f: getattr(p, f) for f in ("dst", "zero_fill_ranges", "remote_stats", "N", "R", "E", "NvS", "K",
                                                        "dup_groups", "dup_loffs", "dup_counts")},
                       "experts_to_copy": etc.to(cuda_device)}) for p in plans]
    rows, cols = 16384, 36864     # 16384*36864*2 B = 1.125 GiB per expert: expert 2 starts at 2.25 GiB
    local = [torch.empty(epn, rows, cols, dtype=torch.bfloat16, device=cuda_device) for _ in range(R)]
    for r in range(R):
        local[r][2].view(torch.int16).copy_(torch.arange(rows * cols, device=cuda_device, dtype=torch.int32).view(rows, cols).to(torch.int16) + r)
    pool, flat = cl.make_pool((epn, rows, cols), torch.bfloat16)
    cl.prefetch(fake, [[(local[r], pool)] for r in range(R)])
    torch.cuda.synchronize()
    cl.check()
    assert torch.equal(pool[0, 2].view(torch.int16), local[1][2].view(torch.int16))
    assert torch.equal(pool[1, 1].view(torch.int16), local[0][2].view(torch.int16))
    assert not pool[0, 0].any() and not pool[1, 2].any()


def test_tensor_factories_single_process(cuda_device):
    """Without a process group the symmetric tensor factories hand out ordinary device memory
    with the same interface (the multi-process path runs in tests/dist_e2e.py)."""
    from moonep_b200.parallel import create_dist_tensor, create_single_owner_tensor
    dt = create_dist_tensor((10, 6), torch.float32)
    assert dt.all.shape == (10, 6) and dt.multicast is None and dt.rows == 10
    dt.local.fill_(2.0)
    assert bool((dt.of_rank(0) == 2.0).all())
    so = create_single_owner_tensor((4, 4), torch.int32)
    assert so.owner == 0 and int(so.tensor.sum()) == 0
    so.destroy()
    dt.destroy()


@pytest.mark.parametrize("R", [1, 4])
def test_push_combine_matches_sum_of_rows(R, cuda_device):
    """Push-combine on emulated ranks: dispatch writes the provenance table, the grouped GEMM
    (identity weights, so its output rows are the dispatched rows) stores every row into its source
    rank's receive area, and the local reduction sums each token's K rows.  The K rows of a token
    are copies of the token, so the exact result is K * token; it must also equal the pull path."""
    from moonep_b200 import routing
    from moonep_b200.ops import grouped_gemm as gg
    from moonep_b200.sim.local_cluster import LocalCluster
    dev = cuda_device
    S, H, K, epn, pad = 96, 256, 4, 4, 128
    E = R * epn
    cl = LocalCluster(S, H, K, E, R, num_sms=4, token_padding=pad, push_combine=True)
    g = torch.Generator().manual_seed(11)
    hidden = [(torch.randn(S, H, generator=g) * 0.5).to(torch.bfloat16).to(dev) for _ in range(R)]
    topk = [routing.lognormal_topk(S, K, E, R, 1.0, 5, r)[0].to(dev) for r in range(R)]
    tpe = [torch.bincount(t.flatten().long(), minlength=E).to(torch.int32) for t in topk]
    wts = [torch.rand(S, K, generator=g).to(dev) for _ in range(R)]
    eye = torch.eye(H, dtype=torch.bfloat16, device=dev).repeat(2 * epn, 1, 1).contiguous()
    for rep in range(2):        # twice: the provenance table is rewritten by every dispatch
        h, w, cus, plans = cl.dispatch(hidden, wts, topk, tpe, zero_copy=True, router_weights_zero_copy=True)
        sink = torch.empty_like(h[0])
        for r in range(R):
            gg.down(h[r], eye, cus[r], sink, push=cl.push_target(r))
        outs, _ = cl.combine_pushed()
        torch.cuda.synchronize()
        cl.check()
        gg.check_status()
        pulled, _ = cl.combine(plans, h, None, zero_copy=True)
        torch.cuda.synchronize()
        for r in range(R):
            want = (hidden[r].float() * K).to(torch.bfloat16)
            assert torch.equal(outs[r], want), f"rank {r}: pushed combine"
            assert torch.equal(pulled[r], want), f"rank {r}: pulled combine"
