"""Pool kernels (prefetch_weight / reduce_grad) on hand-made slot tables.

The planner only ever produces a narrow family of ``experts_to_copy`` tables (hot experts, few slots).
These cases drive the two kernels with tables written by hand instead, along the axes of the
reference's pool tests (tests/test_prefetch.py:1-18, tests/test_grad_reduce.py:249-255, 523-582):
holes, several owners per holder, one expert replicated on every peer, ranks that only send or only
receive, an empty table, random tables over several seeds; payloads from 32 bytes to a megabyte, so that
a copy warp's shared-memory ring is both underfull and wrapped many times within one launch; one to many
CTAs per rank; six tensors in one launch; repeated launches on one cluster.
Every result is compared bit for bit with the CPU oracle (``sim.ops``)."""
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from moonep_b200.sim import ops as simops
from moonep_b200.sim.local_cluster import LocalCluster

pytestmark = pytest.mark.gpu


def table(R, epn, entries):
    t = np.full((R, epn), -1, dtype=np.int64)
    for (d, b), e in entries.items():
        assert e // epn != d, "a slot never holds an expert of its own rank"
        t[d, b] = e
    for d in range(R):
        live = t[d][t[d] >= 0]
        assert len(set(live.tolist())) == len(live), "an expert appears at most once per holder"
    return t


def random_table(R, epn, seed, fill=0.6):
    g = np.random.default_rng(seed)
    t = np.full((R, epn), -1, dtype=np.int64)
    for d in range(R):
        foreign = [e for e in range(R * epn) if e // epn != d]
        picks = g.permutation(foreign)[:epn]
        live = g.random(epn) < fill
        t[d, live] = picks[live]
    return t


def send_only(R, epn):
    """Rank 0 owns every replicated expert: it only sends, the others only receive."""
    return table(R, epn, {(d, b): b for d in range(1, R) for b in range(min(epn, 2))})


def recv_only(R, epn):
    """Only the last rank holds replicas (one from each other rank): it receives and sends nothing."""
    return table(R, epn, {(R - 1, r % epn): r * epn + (epn - 1) for r in range(min(R - 1, epn))})


def everywhere(R, epn):
    """One expert of rank 1 replicated on every other rank: its gradient is the sum of R-1 slots."""
    return table(R, epn, {(d, epn - 1): epn + 1 for d in range(R) if d != 1})


CASES = [
    # name, R, epn, (rows, cols), num_sms, table
    ("empty", 4, 4, (16, 24), 3, lambda R, epn: table(R, epn, {})),
    ("one_slot_last_expert_one_cta", 2, 8, (8, 64), 1, lambda R, epn: table(R, epn, {(1, 0): epn - 1})),
    ("holes_and_two_owners", 4, 4, (40, 24), 4,
     lambda R, epn: table(R, epn, {(0, 1): 5, (0, 3): 14, (2, 0): 1, (2, 2): 13, (3, 3): 0})),
    ("send_only_rank", 4, 3, (24, 40), 2, send_only),
    ("recv_only_rank", 4, 3, (24, 40), 5, recv_only),
    ("one_expert_on_every_peer", 4, 3, (33, 520), 3, everywhere),
    ("ring_wraps_many_times", 2, 2, (512, 1024), 1, lambda R, epn: table(R, epn, {(0, 0): 3, (1, 1): 0, (1, 0): 1})),
    ("fewer_pieces_than_warps", 4, 4, (2, 8), 8, lambda R, epn: random_table(R, epn, 1)),
    ("random_seed_2", 8, 4, (24, 72), 2, lambda R, epn: random_table(R, epn, 2)),
    ("random_seed_3_full", 4, 6, (72, 24), 6, lambda R, epn: random_table(R, epn, 3, fill=1.0)),
    ("random_seed_4_sparse", 8, 3, (128, 136), 3, lambda R, epn: random_table(R, epn, 4, fill=0.3)),
]


def cluster(R, epn, num_sms, dev):
    return LocalCluster(8, 64, 2, R * epn, R, num_sms=num_sms, token_padding=8, device=dev)


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_pool_kernels_on_hand_made_tables(case, cuda_device):
    name, R, epn, (rows, cols), num_sms, make = case
    etc = make(R, epn)
    dev = cuda_device
    cl = cluster(R, epn, num_sms, dev)
    cp = SimpleNamespace(experts_to_copy=etc, E=R * epn, R=R)
    plans = [SimpleNamespace(experts_to_copy=torch.from_numpy(etc).to(torch.int32).to(dev)) for _ in range(R)]
    g = torch.Generator().manual_seed(11)
    shapes = {"gate": (rows, cols), "up": (rows, cols), "down": (cols, rows)}

    # ---- prefetch: two launches with different weights (the second must overwrite the first)
    pools, flats = {}, {}
    for n, shp in shapes.items():
        pools[n], flats[n] = cl.make_pool((epn, *shp), torch.bfloat16, pad_elems=8)
        flats[n].fill_(-3.0)
    exp = {n: [torch.full((epn, *shp), -3.0, dtype=torch.bfloat16) for _ in range(R)] for n, shp in shapes.items()}
    for launch in range(2):
        local = {n: [torch.randn(epn, *shp, generator=g).to(torch.bfloat16) for _ in range(R)] for n, shp in shapes.items()}
        pairs = [[(local[n][r].to(dev), pools[n]) for n in shapes] for r in range(R)]
        cl.prefetch(plans, pairs)
        torch.cuda.synchronize()
        cl.check()
        for n in shapes:
            simops.prefetch(cp, local[n], exp[n])
            for r in range(R):
                assert torch.equal(pools[n][r].cpu(), exp[n][r]), f"{name}: launch {launch}, {n} slots of rank {r}"
            per = epn * rows * cols
            assert (flats[n].cpu().view(R, per + 8)[:, per:] == -3.0).all(), f"{name}: gap between ranks overwritten"

    # ---- reduce_grad: three launches, slots refilled in between (bitwise: fixed summation order)
    rpools = {n: cl.make_pool((epn, *shp), torch.float32, pad_elems=4)[0] for n, shp in shapes.items()}
    lg = {n: [torch.randn(epn, *shp, generator=g) for _ in range(R)] for n, shp in shapes.items()}
    lgd = {n: [x.to(dev) for x in lg[n]] for n in shapes}
    pairs = [[(lgd[n][r], rpools[n]) for n in shapes] for r in range(R)]
    for launch in range(3):
        rb = {n: [torch.randn(epn, *shp, generator=g) for _ in range(R)] for n, shp in shapes.items()}
        for n in shapes:
            for r in range(R):
                rpools[n][r].copy_(rb[n][r])
        cl.reduce_grad(plans, pairs)
        torch.cuda.synchronize()
        cl.check()
        for n in shapes:
            simops.reduce_grad(cp, lg[n], rb[n])
            for r in range(R):
                assert torch.equal(lgd[n][r].cpu(), lg[n][r]), f"{name}: launch {launch}, {n} grads of rank {r}"
                assert torch.equal(rpools[n][r].cpu(), rb[n][r]), f"{name}: launch {launch}, {n} slots of rank {r}"


def test_six_tensors_send_only_and_wrapped_ring(cuda_device):
    """Weights and block scales in one launch, from a rank that only sends, with payloads of unequal
    size (the piece list of one slot spans six tensors) and one CTA per rank (rings wrap)."""
    R, epn, dev = 3, 4, cuda_device
    etc = send_only(R, epn)
    cl = cluster(R, epn, 1, dev)
    cp = SimpleNamespace(experts_to_copy=etc, E=R * epn, R=R)
    plans = [SimpleNamespace(experts_to_copy=torch.from_numpy(etc).to(torch.int32).to(dev)) for _ in range(R)]
    g = torch.Generator().manual_seed(3)
    shapes = [((256, 448), torch.uint8), ((256, 448), torch.uint8), ((448, 256), torch.int8),
              ((256, 16), torch.uint8), ((256, 16), torch.uint8), ((448, 16), torch.uint8)]
    local, pools = [], []
    for shp, dt in shapes:
        local.append([torch.randint(0, 120, (epn, *shp), generator=g).to(dt) for _ in range(R)])
        pool, flat = cl.make_pool((epn, *shp), dt, pad_elems=32)
        flat.fill_(9)
        pools.append(pool)
    pairs = [[(local[i][r].to(dev), pools[i]) for i in range(6)] for r in range(R)]
    for _ in range(2):
        cl.prefetch(plans, pairs)
    torch.cuda.synchronize()
    cl.check()
    for i, (shp, dt) in enumerate(shapes):
        exp = [torch.full((epn, *shp), 9, dtype=dt) for _ in range(R)]
        simops.prefetch(cp, local[i], exp)
        for r in range(R):
            assert torch.equal(pools[i][r].cpu(), exp[r]), f"tensor {i}: slots of rank {r} differ"


def test_pool_kernels_run_beside_token_kernels(cuda_device):
    """prefetch_weight / reduce_grad on a second stream while dispatch / combine of the same cluster run on
    the first: the two families keep separate barrier words, so neither order of arrival may disturb the
    other.  Every result is compared with the oracle after each of several rounds."""
    from gpu_helpers import run_case
    R, epn, S, K, H = 4, 4, 200, 6, 64
    cl, cp, plans, cus, hidden, weights, topk, tpe, oh, ow = run_case(S, K, epn, H, R, 4, 16, "biased", sigma=2.0)
    assert (cp.experts_to_copy >= 0).any(), "case must produce redundant experts"
    dev = cuda_device
    g = torch.Generator().manual_seed(21)
    rows, cols = 256, 136
    names = ("gate", "up", "down")
    pools = {n: cl.make_pool((epn, rows, cols), torch.bfloat16)[0] for n in names}
    rpools = {n: cl.make_pool((epn, rows, cols), torch.float32)[0] for n in names}
    ys = []
    for d in range(R):
        y = torch.zeros(cp.NvS, H, dtype=torch.bfloat16)
        y[:] = ((torch.arange(cp.NvS) % 7) + 1)[:, None].to(torch.bfloat16)
        ys.append(y.to(dev))
    wd = [w.to(dev) for w in ow]
    eo, _ = simops.combine(cp, [y.cpu().float() for y in ys], [w.cpu().view(torch.int32).float() for w in ow])
    lg = {n: [torch.randn(epn, rows, cols, generator=g) for _ in range(R)] for n in names}
    lgd = {n: [x.to(dev) for x in lg[n]] for n in names}
    side = torch.cuda.Stream()
    for it in range(4):
        local = {n: [torch.randn(epn, rows, cols, generator=g).to(torch.bfloat16) for _ in range(R)] for n in names}
        rb = {n: [torch.randn(epn, rows, cols, generator=g) for _ in range(R)] for n in names}
        for n in names:
            for r in range(R):
                rpools[n][r].copy_(rb[n][r])
        ppairs = [[(local[n][r].to(dev), pools[n]) for n in names] for r in range(R)]
        rpairs = [[(lgd[n][r], rpools[n]) for n in names] for r in range(R)]
        torch.cuda.synchronize()
        with torch.cuda.stream(side):
            if it % 2 == 0:
                cl.prefetch(plans, ppairs)
                cl.reduce_grad(plans, rpairs)
        outs, _ = cl.combine(plans, ys, wd)
        cl.dispatch([h.to(dev) for h in hidden], None, plans=plans)
        if it % 2 == 1:       # the other order of issue
            with torch.cuda.stream(side):
                cl.prefetch(plans, ppairs)
                cl.reduce_grad(plans, rpairs)
        torch.cuda.synchronize()
        cl.check()
        for r in range(R):
            assert torch.equal(outs[r].cpu().float(), eo[r].to(torch.bfloat16).float()), f"round {it}: combine of rank {r}"
        for n in names:
            exp = [pools[n][r].cpu().clone() for r in range(R)]
            simops.prefetch(cp, local[n], exp)
            simops.reduce_grad(cp, lg[n], rb[n])
            for r in range(R):
                assert torch.equal(pools[n][r].cpu(), exp[r]), f"round {it}: {n} prefetch slots of rank {r}"
                assert torch.equal(lgd[n][r].cpu(), lg[n][r]), f"round {it}: {n} reduced grads of rank {r}"
                assert torch.equal(rpools[n][r].cpu(), rb[n][r]), f"round {it}: {n} reduce slots of rank {r}"
