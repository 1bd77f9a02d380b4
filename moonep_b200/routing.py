"""Synthetic router outputs for tests and benchmarks.

Two generators:

* ``lognormal_topk``: the reference's benchmark generator
  (tests/generate_topk_routing.py:6-44) -- ``sigma == 0`` gives a round-robin,
  perfectly balanced table (every token visits every rank once when K == R);
  otherwise expert popularity is lognormal(sigma) shared by all ranks and each
  token draws K distinct experts.
* ``softmax_topk``: per-token N(0,1) logits plus ``scale`` x a per-expert N(0,1)
  bias shared by all ranks; top-k of the softmax, with the renormalised
  probabilities as route weights.

``maxvio = max_e(T_e / mean_e T_e) - 1`` over the whole EP group
(README.md:15-17 of the reference); ``solve_scale_for_maxvio`` bisects the skew
parameter on a log scale until the realised value is within 2 % of the target.
"""

from __future__ import annotations

import math

import torch


def lognormal_topk(S, K, E, R, sigma, seed, rank, device="cpu"):
    g_shared = torch.Generator(device=device).manual_seed(seed)
    g_local = torch.Generator(device=device).manual_seed(rank)
    if sigma == 0.0:
        epn = E // R
        t = torch.arange(S, device=device)[:, None]
        k = torch.arange(K, device=device)[None, :]
        perm = torch.randperm(epn, device=device, generator=g_local)
        topk = ((t + k) % R) * epn + perm[((t // R) + k) % epn]
    else:
        pop = torch.exp(torch.normal(0.0, sigma, size=(E,), device=device, generator=g_shared))
        topk = torch.multinomial(pop[None, :].expand(S, E), K, replacement=False, generator=g_local)
    topk = topk.to(torch.int32).contiguous()
    tpe = torch.bincount(topk.flatten().long(), minlength=E).to(torch.int32)
    return topk, tpe


def softmax_topk(S, K, E, scale, seed, rank, device="cpu"):
    """Returns ``(topk[S,K] int32, weights[S,K] fp32, tpe[E] int32)``."""
    g_shared = torch.Generator(device=device).manual_seed(seed)
    g_local = torch.Generator(device=device).manual_seed(seed * 1000003 + rank + 1)
    bias = torch.randn(E, device=device, generator=g_shared)
    logits = torch.randn(S, E, device=device, generator=g_local) + scale * bias[None, :]
    probs = torch.softmax(logits, dim=-1)
    w, topk = torch.topk(probs, K, dim=-1)
    w = (w / w.sum(dim=-1, keepdim=True)).float().contiguous()
    topk = topk.to(torch.int32).contiguous()
    tpe = torch.bincount(topk.flatten().long(), minlength=E).to(torch.int32)
    return topk, w, tpe


def maxvio(tpe_total: torch.Tensor) -> float:
    t = tpe_total.double()
    return float(t.max() / t.mean() - 1.0)


def _maxvio_for_scale(S, K, E, R, scale, seed):
    tot = torch.zeros(E, dtype=torch.int64)
    for r in range(R):
        _, _, tpe = softmax_topk(S, K, E, scale, seed, r)
        tot += tpe.long()
    return maxvio(tot)


def solve_scale_for_maxvio(target, S, K, E, R, seed=0, iters=40):
    """Skew scale whose realised group-wide maxvio is closest to ``target``.

    Returns ``(scale, realised)``.  Targets below the sampling-noise floor (about
    0.08-0.10 for E=256, S=4096, R=8) return scale 0 and the floor value."""
    floor = _maxvio_for_scale(S, K, E, R, 0.0, seed)
    if target <= floor:
        return 0.0, floor
    lo, hi = 1e-4, 4.0
    best = (0.0, floor)
    for _ in range(iters):
        mid = math.sqrt(lo * hi)
        mv = _maxvio_for_scale(S, K, E, R, mid, seed)
        if abs(mv - target) < abs(best[1] - target):
            best = (mid, mv)
        if abs(mv - target) <= max(0.02 * target, 0.005):
            break
        if mv < target:
            lo = mid
        else:
            hi = mid
    return best


# synthetic patterns used by the kernel tests (cf. tests/kernel_test_utils.py:94-113)
def pattern_topk(pattern, S, K, E, R, rank):
    epn = E // R
    s = torch.arange(S)[:, None]
    k = torch.arange(K)[None, :]
    if pattern == "all_local":
        topk = rank * epn + ((s + k) % epn)
    elif pattern == "all_remote":
        topk = ((rank + 1) % R) * epn + ((s + k) % epn)
    elif pattern == "single_expert":
        topk = torch.zeros((S, K), dtype=torch.long)
    elif pattern == "duplicate_topk":
        topk = torch.full((S, K), ((rank + 1) % R) * epn, dtype=torch.long)
    else:
        raise ValueError(f"unknown routing pattern {pattern!r}")
    topk = topk.to(torch.int32).contiguous()
    tpe = torch.bincount(topk.flatten().long(), minlength=E).to(torch.int32)
    return topk, tpe
