"""CPU tests of the planner oracle and the emulated data movement (no GPU)."""
import numpy as np
import pytest
import torch
from hypothesis import given, settings, strategies as st

from moonep_b200 import routing
from moonep_b200.sim import plan_cluster, check_invariants, ops


def _topk_all(R, S, K, E, gen):
    return np.stack([gen(r)[0].numpy() for r in range(R)])


@pytest.mark.parametrize("scale_target", [0.0, 0.5, 2.0])
def test_baseline_cpu_config(scale_target):
    """R=8, S=512, K=8, E=64, token_padding=16, softmax top-k with skew bias."""
    R, S, K, E, pad = 8, 512, 8, 64, 16
    scale, realised = routing.solve_scale_for_maxvio(scale_target, S, K, E, R, seed=0) if scale_target else (0.0, 0.0)
    outs = [routing.softmax_topk(S, K, E, scale, 0, r) for r in range(R)]
    topk = np.stack([o[0].numpy() for o in outs])
    cp = plan_cluster(topk, E, pad)
    check_invariants(cp)
    H = 32
    g = torch.Generator().manual_seed(1)
    hidden = [torch.randn(S, H, generator=g) for _ in range(R)]
    weights = [o[1] for o in outs]
    hn, wn = ops.dispatch(cp, hidden, weights)
    # every rank received exactly S*K real rows
    for d in range(R):
        real = ops.expert_of_slot(cp, d) >= 0
        assert int(real.sum()) == S * K
        assert not torch.isnan(hn[d][torch.from_numpy(real)]).any()
    # the "FFN" scales each row by its route weight; combine must give sum_k p_k * x
    y = [torch.nan_to_num(hn[d]) * torch.nan_to_num(wn[d])[:, None] for d in range(R)]
    out, wsk = ops.combine(cp, y, wn)
    for r in range(R):
        assert torch.equal(wsk[r], weights[r])
        expect = hidden[r] * weights[r].sum(dim=1, keepdim=True)
        assert torch.allclose(out[r], expect, rtol=1e-5, atol=1e-5)
    # weight grads: redundancy must not change the reduced result
    epn = E // R
    Hp = 4
    slot_e = [ops.expert_of_slot(cp, d) for d in range(R)]
    ref = [torch.zeros(epn, H, Hp) for _ in range(R)]
    local = [torch.zeros(epn, H, Hp) for _ in range(R)]
    red = [torch.zeros(epn, H, Hp) for _ in range(R)]
    dy = [torch.randn(cp.NvS, Hp, generator=g) for _ in range(R)]
    for d in range(R):
        for g_ in range(2 * epn):
            e = d * epn + g_ if g_ < epn else int(cp.experts_to_copy[d, g_ - epn])
            if e < 0:
                continue
            rows = torch.from_numpy(slot_e[d] == e)
            contrib = hn[d][rows].T @ dy[d][rows]
            ref[e // epn][e % epn] += contrib
            (local[d] if g_ < epn else red[d])[g_ % epn] += contrib
    ops.reduce_grad(cp, local, red)
    for r in range(R):
        assert torch.allclose(local[r], ref[r], rtol=1e-4, atol=1e-4)
        assert not red[r].any()


@pytest.mark.parametrize("pattern", ["all_local", "all_remote", "single_expert", "duplicate_topk"])
@pytest.mark.parametrize("R", [1, 2, 4])
def test_patterns(pattern, R):
    S, K, epn, pad = 33, 4, 3, 8
    E = R * epn
    topk = np.stack([routing.pattern_topk(pattern, S, K, E, R, r)[0].numpy() for r in range(R)])
    cp = plan_cluster(topk, E, pad)
    check_invariants(cp)


@pytest.mark.parametrize("sigma", [0.0, 0.5, 1.0, 5.0])
def test_lognormal(sigma):
    R, S, K, E = 8, 256, 8, 64
    topk = np.stack([routing.lognormal_topk(S, K, E, R, sigma, 42, r)[0].numpy() for r in range(R)])
    cp = plan_cluster(topk, E, 128)
    check_invariants(cp)
    if sigma == 0.0:
        assert (cp.experts_to_copy < 0).all()


@settings(max_examples=60, deadline=None)
@given(R=st.sampled_from([1, 2, 3, 4, 8]), epn=st.integers(1, 5), S=st.integers(1, 40),
       K=st.integers(1, 6), pad=st.sampled_from([1, 4, 16]), seed=st.integers(0, 10_000),
       hot=st.floats(0.0, 1.0))
def test_planner_properties(R, epn, S, K, pad, seed, hot):
    E = R * epn
    rng = np.random.default_rng(seed)
    p = rng.random(E) ** (1 + 8 * hot)
    p /= p.sum()
    topk = rng.choice(E, size=(R, S, K), p=p)
    cp = plan_cluster(topk, E, pad)
    check_invariants(cp)
    # duplicate encoding: exactly one non-negative entry per (token, destination rank)
    dest = cp.dst_raw // cp.NvS
    for r in range(R):
        for s in range(S):
            row = slice(s * K, (s + 1) * K)
            prim = dest[r, row][cp.dst[r, row] >= 0]
            assert len(set(prim.tolist())) == len(prim) == len(set(dest[r, row].tolist()))


from shape_cases import case_params, case_id, SHAPE_CASES  # noqa: E402


@pytest.mark.parametrize("p", case_params(), ids=case_id)
def test_shape_list_on_the_oracle(p):
    """Every shape of the shared list satisfies the planner invariants, fits the buffer geometry
    and moves tokens consistently through the emulated dispatch / combine."""
    from gpu_helpers import make_topk
    from moonep_b200.geometry import Geometry
    c, R = p
    E = R * c.epn
    topk, tpe = make_topk(c.routing, c.S, c.K, E, R, c.seed, c.sigma)
    cp = plan_cluster(np.stack([t.numpy() for t in topk]), E, c.pad)
    check_invariants(cp)
    geo = Geometry.make(c.S, c.H, c.K, E, R, c.pad, 1)
    assert geo.NvS == cp.NvS
    for r in range(R):
        assert torch.equal(torch.from_numpy(np.bincount(topk[r].numpy().ravel(), minlength=E)).int(), tpe[r])
    if c.S * c.K * R <= 4096:        # identity round trip on the small shapes
        hidden = [torch.arange(c.S, dtype=torch.float32)[:, None].repeat(1, 4) + 1000 * r for r in range(R)]
        hn, _ = ops.dispatch(cp, hidden, None)
        out, _ = ops.combine(cp, [torch.nan_to_num(h) for h in hn], None)
        for r in range(R):       # combine is a plain sum over a token's K rows, duplicates included
            assert torch.equal(out[r], hidden[r] * float(c.K))


def test_shape_list_reaches_every_planner_regime():
    """The list must keep covering: E above one thread block, E*R above the fast planner's table
    limit, padding of 1, padding above every segment, K=1, one token, and all four synthetic
    routings (a guard against trimming the list)."""
    names = {c.name for c in SHAPE_CASES}
    assert any(c.epn > 1024 for c in SHAPE_CASES)
    assert any(c.epn * c.max_R * c.max_R > 8192 for c in SHAPE_CASES)
    assert any(c.pad == 1 for c in SHAPE_CASES) and any(c.pad > c.S * c.K for c in SHAPE_CASES)
    assert any(c.K == 1 for c in SHAPE_CASES) and any(c.S == 1 for c in SHAPE_CASES)
    assert {"all_local", "all_remote", "single_expert", "duplicate_topk"} <= {c.routing for c in SHAPE_CASES}
    assert len(names) == len(SHAPE_CASES)


def _plans_from_oracle(cp):
    """MoonEPCommPlan objects (CPU tensors) for every rank of an oracle plan."""
    from moonep_b200 import MoonEPCommPlan
    R, epn, NvS = cp.R, cp.E // cp.R, cp.NvS
    i32 = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(torch.int32).contiguous()  # noqa: E731
    z = lambda *s: torch.zeros(*s, dtype=torch.int32)  # noqa: E731
    return [MoonEPCommPlan(dst=i32(cp.dst[r]), experts_to_copy=i32(cp.experts_to_copy),
                           zero_fill_ranges=i32(cp.zero_fill_ranges[r]), remote_stats=i32(cp.remote_stats[r]),
                           N=cp.dst.shape[1], R=R, E=cp.E, NvS=NvS, K=cp.K,
                           dup_groups=z(NvS, 3), dup_loffs=z(NvS), dup_counts=z(2)) for r in range(R)]


def test_plan_fingerprints_agree_and_catch_divergence():
    """The cross-rank plan check accepts the oracle's plans and names each kind of divergence."""
    from moonep_b200.plan import plan_fingerprint, compare_fingerprints
    R, S, K, epn = 4, 64, 4, 4
    topk = np.stack([routing.lognormal_topk(S, K, R * epn, R, 2.0, 7, r)[0].numpy() for r in range(R)])
    cp = plan_cluster(topk, R * epn, 16)
    assert (cp.experts_to_copy >= 0).any()
    plans = _plans_from_oracle(cp)
    fps = [plan_fingerprint(p, r) for r, p in enumerate(plans)]
    assert compare_fingerprints(fps) == []
    # a rank whose slot table differs
    bad = plans[2].clone()
    bad.experts_to_copy[0, -1] = 1
    errs = compare_fingerprints(fps[:2] + [plan_fingerprint(bad, 2)] + fps[3:])
    assert any("experts_to_copy differs" in e for e in errs)
    # a rank that routes one row to another destination: two ranks no longer receive S*K rows
    bad = plans[1].clone()
    raw = int(bad.dst[0]) if int(bad.dst[0]) >= 0 else -int(bad.dst[0]) - 1
    bad.dst[0] = ((raw // cp.NvS + 1) % R) * cp.NvS + raw % cp.NvS
    errs = compare_fingerprints([fps[0], plan_fingerprint(bad, 1)] + fps[2:])
    assert sum("receives" in e for e in errs) == 2
    # statistics that do not match the table
    bad = plans[0].clone()
    bad.remote_stats[0] += 1
    assert any("remote_stats" in e for e in compare_fingerprints([plan_fingerprint(bad, 0)] + fps[1:]))
    # plans survive pickling (debug dumps)
    import pickle
    again = pickle.loads(pickle.dumps(plans[0]))
    assert torch.equal(again.dst, plans[0].dst) and again.NvS == plans[0].NvS


def test_workload_report_counts():
    """The offline workload report: counters agree with the plan they are computed from."""
    from moonep_b200.sim.report import report, workload
    R, S, K, E, H, Hp = 4, 128, 4, 16, 256, 128
    rep = report(R, S, K, E, H, Hp, 2.0, token_padding=16)
    assert rep["redundant_slots"] == sum(rep["slots_sent_per_owner"]) and rep["max_slots_sent"] >= 1
    assert 1.0 <= rep["distinct_dest_ranks_per_token"] <= min(K, R)
    assert rep["NvS"] == -(-(S * K + 15 * 2 * (E // R)) // 16) * 16      # capacity rule, rounded up to the padding
    # all-local routing: nothing crosses a link, K-1 of every K rows are duplicates
    topk = np.stack([routing.pattern_topk("all_local", S, K, E, R, r)[0].numpy() for r in range(R)])
    w = workload(plan_cluster(topk, E, 16), H, Hp)
    assert w["dispatch_egress_MB_max"] == 0 and w["dispatch_us_at_link"] == 0
    assert w["duplicate_rows_pct"] == 75.0 and w["redundant_slots"] == 0 and w["tokens_off_home_pct"] == 0
    # all-remote routing: every token sends exactly one row to its neighbour
    topk = np.stack([routing.pattern_topk("all_remote", S, K, E, R, r)[0].numpy() for r in range(R)])
    w = workload(plan_cluster(topk, E, 16), H, Hp)
    assert w["dispatch_egress_MB_max"] == round(S * H * 2 / 1e6, 1)


@pytest.mark.parametrize("target", [0.5, 1.0, 2.0, 3.0])
def test_skew_solver_hits_the_requested_maxvio(target):
    """The routing generator's skew scale is solved so that the realised group-wide
    maxvio = max_e(T_e) / mean_e(T_e) - 1 lands on the target; below the sampling-noise floor
    it reports the floor instead."""
    R, S, K, E = 8, 512, 8, 64
    scale, realised = routing.solve_scale_for_maxvio(target, S, K, E, R, seed=0)
    assert scale > 0 and abs(realised - target) <= max(0.05 * target, 0.02)
    tot = sum(routing.softmax_topk(S, K, E, scale, 0, r)[2].long() for r in range(R))
    assert abs(routing.maxvio(tot) - realised) < 1e-9
    floor_scale, floor = routing.solve_scale_for_maxvio(0.01, S, K, E, R, seed=0)
    assert floor_scale == 0.0 and 0.0 < floor < 0.5
    # weights are a normalised top-k distribution and topk ids are distinct per token
    topk, w, tpe = routing.softmax_topk(S, K, E, scale, 0, 3)
    assert torch.allclose(w.sum(dim=1), torch.ones(S), atol=1e-5) and int(tpe.sum()) == S * K
    assert all(len(set(row.tolist())) == K for row in topk[:32])


def test_update_mask_names_exactly_the_unreplicated_local_experts():
    """The mask that decides which experts the weight-gradient GEMM may update in its epilogue: on real plans
    of the oracle, a local expert is masked in iff no rank holds a replica of it; slots are never masked in."""
    import torch
    from moonep_b200.moe_layer import update_mask
    R, epn, S, K = 4, 6, 300, 4
    E = R * epn
    seen_replica = False
    for seed in range(5):
        topk = np.stack([routing.lognormal_topk(S, K, E, R, 2.0, seed, r)[0].numpy() for r in range(R)])
        cp = plan_cluster(topk, E, 16)
        etc = torch.from_numpy(np.asarray(cp.experts_to_copy)).to(torch.int32)
        replicated = {int(e) for e in etc.flatten().tolist() if e >= 0}
        seen_replica |= bool(replicated)
        for r in range(R):
            m = update_mask(etc, r, epn)
            assert m.dtype == torch.int32 and m.shape == (2 * epn,)
            want = [0 if (r * epn + g) in replicated else 1 for g in range(epn)] + [0] * epn
            assert m.tolist() == want, f"seed {seed} rank {r}"
    assert seen_replica, "the routing must produce replicas for this test to mean anything"
    # preallocated work tensors are reused correctly across calls with different tables
    mask, hit, ones = torch.zeros(2 * epn, dtype=torch.int32), torch.zeros(epn + 1, dtype=torch.int32), torch.ones(R * epn, dtype=torch.int32)
    a = torch.full((R, epn), -1, dtype=torch.int32); a[1, 0] = 2
    assert update_mask(a, 0, epn, mask, hit, ones).tolist() == [1, 1, 0, 1, 1, 1] + [0] * epn
    b = torch.full((R, epn), -1, dtype=torch.int32)
    assert update_mask(b, 0, epn, mask, hit, ones).tolist() == [1] * epn + [0] * epn
