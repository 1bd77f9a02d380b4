"""Shared helpers for the GPU tests: run a routing case through the single-GPU LocalCluster
and compare every output with the CPU oracle."""
import numpy as np
import torch

from moonep_b200 import routing
from moonep_b200.sim import plan_cluster, dup_table_from_arrays, ops as simops
from moonep_b200.sim.local_cluster import LocalCluster


def make_topk(routing_kind, S, K, E, R, seed=42, sigma=1.0):
    outs = []
    for r in range(R):
        if routing_kind == "balanced":
            outs.append(routing.lognormal_topk(S, K, E, R, 0.0, seed, r))
        elif routing_kind == "biased":
            outs.append(routing.lognormal_topk(S, K, E, R, sigma, seed, r))
        elif routing_kind == "random":
            g = torch.Generator().manual_seed(seed * 131 + r)
            t = torch.randint(0, E, (S, K), dtype=torch.int32, generator=g)
            outs.append((t, torch.bincount(t.flatten().long(), minlength=E).to(torch.int32)))
        else:
            outs.append(routing.pattern_topk(routing_kind, S, K, E, R, r))
    return [o[0] for o in outs], [o[1] for o in outs]


def traceable_hidden(S, H, rank):
    """Row s of rank r carries (s, r) in its first lanes and a ramp elsewhere: exact in bf16
    for s < 256*... so we use int16 bit patterns instead of float values."""
    v = torch.zeros(S, H, dtype=torch.int16)
    v[:, 0] = torch.arange(S, dtype=torch.int32).to(torch.int16)
    v[:, 1] = rank
    v[:, 2:] = ((torch.arange(S)[:, None] * 7 + torch.arange(H - 2)[None, :] * 3 + rank) % 251).to(torch.int16)
    return v.view(torch.bfloat16)


def check_plans(plans, cus, cp, R):
    for r in range(R):
        p = plans[r]
        assert torch.equal(p.dst.cpu().long(), torch.from_numpy(cp.dst[r])), f"rank {r}: dst mismatch"
        assert torch.equal(cus[r].cpu().long(), torch.from_numpy(cp.cu_seqlens[r])), f"rank {r}: cu_seqlens mismatch"
        assert torch.equal(p.experts_to_copy.cpu().long(), torch.from_numpy(cp.experts_to_copy)), f"rank {r}: experts_to_copy"
        assert torch.equal(p.zero_fill_ranges.cpu().long(), torch.from_numpy(cp.zero_fill_ranges[r])), f"rank {r}: zero_fill"
        assert torch.equal(p.remote_stats.cpu().long(), torch.from_numpy(cp.remote_stats[r])), f"rank {r}: remote_stats"
        got = dup_table_from_arrays(p.dup_groups.cpu().numpy(), p.dup_loffs.cpu().numpy(), p.dup_counts.cpu().numpy())
        want = {k: tuple(sorted(v)) for k, v in cp.dup_tables[r].items()}
        assert got == want, f"rank {r}: duplicate groups differ ({len(got)} vs {len(want)})"
        assert int(p.dup_counts[1]) == sum(len(v) for v in want.values())


def defined_rows(cp, d):
    """Boolean mask of rows whose content dispatch defines (real + padding)."""
    m = np.zeros(cp.NvS, dtype=bool)
    start = 0
    for g in range(cp.cu_seqlens.shape[1]):
        end = int(cp.cu_seqlens[d, g])
        m[start:end] = True
        start = end
    return torch.from_numpy(m)


def run_case(S, K, epn, H, R, num_sms, token_padding, routing_kind, seed=42, sigma=1.0, with_weights=True,
             device="cuda:0"):
    E = R * epn
    topk, tpe = make_topk(routing_kind, S, K, E, R, seed, sigma)
    cp = plan_cluster(np.stack([t.numpy() for t in topk]), E, token_padding)
    cl = LocalCluster(S, H, K, E, R, num_sms=num_sms, token_padding=token_padding, device=device)
    assert cl.geo.NvS == cp.NvS
    hidden = [traceable_hidden(S, H, r) for r in range(R)]
    weights = [(torch.arange(S * K, dtype=torch.int32) + r * S * K + 1).view(torch.float32).reshape(S, K) for r in range(R)]
    dev = torch.device(device)
    # poison the shards so missing writes show
    for s in cl._states:
        s.hidden_local.view(torch.int16).fill_(0x5555)
        s.weights_local.view(torch.int32).fill_(0x55555555)
    oh, ow, cus, plans = cl.dispatch([h.to(dev) for h in hidden], [w.to(dev) for w in weights] if with_weights else None,
                                     [t.to(dev) for t in topk], [t.to(dev) for t in tpe])
    torch.cuda.synchronize()
    cl.check()
    check_plans(plans, cus, cp, R)
    eh, ew = simops.dispatch(cp, [h.view(torch.int16).float() for h in hidden],
                             [w.view(torch.int32).float() for w in weights] if with_weights else None, fill=-1.0)
    for d in range(R):
        m = defined_rows(cp, d)
        got = oh[d].cpu().view(torch.int16).float()
        assert torch.equal(got[m], eh[d][m]), f"rank {d}: dispatched rows differ"
        if with_weights:
            gw = ow[d].cpu().view(torch.int32).float()
            assert torch.equal(gw[m], ew[d][m]), f"rank {d}: dispatched weights differ"
    return cl, cp, plans, cus, hidden, weights, topk, tpe, oh, ow
