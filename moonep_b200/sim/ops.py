"""fp32 torch emulation of dispatch / combine / prefetch / reduce_grad on CPU.

All ranks live in one process as lists indexed by rank.  These functions define
the data-movement semantics the device kernels are tested against
(reference behaviour: moonep/dispatch.py:268-692, combine.py:403-407,
combine_prologue.py:41-484, prefetch.py:316-460, grad_reduce.py:296-389).
"""

from __future__ import annotations

import numpy as np
import torch

from .planner import ClusterPlan


def dispatch(cp: ClusterPlan, hidden, weights=None, fill=float("nan")):
    """``hidden[r]``: [S, H]; ``weights[r]``: [S, K] or None.

    Returns ``(hidden_nvsh[r] [NvS,H], weights_nvs[r] [NvS] | None)``.  Real rows and
    padding rows (zeros) are defined; the tail beyond ``cu_seqlens[-1]`` holds
    ``fill``."""
    R, NvS, K = cp.R, cp.NvS, cp.K
    H = hidden[0].shape[1]
    out_h = [torch.full((NvS, H), fill, dtype=hidden[0].dtype) for _ in range(R)]
    out_w = [torch.full((NvS,), fill, dtype=torch.float32) for _ in range(R)] if weights is not None else None
    for d in range(R):
        start = 0
        for g in range(cp.cu_seqlens.shape[1]):
            p0, n = (int(x) for x in cp.zero_fill_ranges[d, g])
            if n:
                out_h[d][p0:p0 + n] = 0
                if out_w is not None:
                    out_w[d][p0:p0 + n] = 0
    for r in range(R):
        raw = torch.from_numpy(cp.dst_raw[r])
        dest = raw // NvS
        loff = raw % NvS
        tok = torch.arange(raw.numel()) // K
        for d in range(R):
            m = dest == d
            out_h[d][loff[m]] = hidden[r][tok[m]]
            if out_w is not None:
                out_w[d][loff[m]] = weights[r].reshape(-1)[m]
    return out_h, out_w


def combine(cp: ClusterPlan, hidden_nvsh, weights_nvs=None):
    """Unweighted sum of each token's K rows.  Rows of one token that sit on the same
    rank are first summed in fp32 and rounded to the payload dtype once (the
    destination's local pre-reduction); the per-rank partial sums are then added in
    fp32 in ascending ``k`` order of their primaries and rounded once more."""
    R, NvS, K, S = cp.R, cp.NvS, cp.K, cp.S
    dt = hidden_nvsh[0].dtype
    H = hidden_nvsh[0].shape[1]
    outs, wouts = [], []
    for r in range(R):
        raw = torch.from_numpy(cp.dst_raw[r]).reshape(S, K)
        dest = raw // NvS
        loff = raw % NvS
        isdup = torch.from_numpy(cp.dst[r] < 0).reshape(S, K)
        acc = torch.zeros(S, H, dtype=torch.float32)
        for k in range(K):           # primaries in ascending k
            part = torch.zeros(S, H, dtype=torch.float32)
            prim = ~isdup[:, k]
            for k2 in range(k, K):   # this primary plus its duplicates on the same rank
                same = prim & (dest[:, k2] == dest[:, k]) & ((k2 == k) | isdup[:, k2])
                if not same.any():
                    continue
                rows = torch.zeros(S, H, dtype=torch.float32)
                for d in range(R):
                    m = same & (dest[:, k2] == d)
                    if m.any():
                        rows[m] = hidden_nvsh[d][loff[m, k2]].float()
                part += rows
            n_on_rank = (prim[:, None] & (dest == dest[:, k:k + 1])).sum(dim=1)
            part_rounded = torch.where((n_on_rank > 1)[:, None], part.to(dt).float(), part)
            acc += torch.where(prim[:, None], part_rounded, torch.zeros_like(part_rounded))
        outs.append(acc.to(dt))
        if weights_nvs is not None:
            w = torch.zeros(S, K, dtype=torch.float32)
            for d in range(R):
                m = dest == d
                w[m] = weights_nvs[d][loff[m]]
            wouts.append(w)
    return outs, (wouts if weights_nvs is not None else None)


def prefetch(cp: ClusterPlan, local_weights, pools):
    """``local_weights[r]``: [epn, ...]; ``pools[r]``: [epn, ...] prefetch slots of rank r
    (modified in place).  Slot ``b`` of rank ``d`` receives expert ``experts_to_copy[d,b]``
    from its home rank."""
    epn = cp.E // cp.R
    for d in range(cp.R):
        for b in range(epn):
            e = int(cp.experts_to_copy[d, b])
            if e >= 0:
                pools[d][b].copy_(local_weights[e // epn][e % epn])


def reduce_grad(cp: ClusterPlan, local_grads, reduce_bufs):
    """``local_grads[r] += sum`` of the slots holding r's experts, in ascending
    ``(rank, slot)`` order (fixed order => bitwise reproducible); afterwards every rank
    zeroes its own consumed slots.  Unused slots are left untouched."""
    epn = cp.E // cp.R
    for d in range(cp.R):
        for b in range(epn):
            e = int(cp.experts_to_copy[d, b])
            if e >= 0:
                local_grads[e // epn][e % epn] += reduce_bufs[d][b]
    for d in range(cp.R):
        for b in range(epn):
            if int(cp.experts_to_copy[d, b]) >= 0:
                reduce_bufs[d][b].zero_()


def expert_of_slot(cp: ClusterPlan, d: int) -> np.ndarray:
    """Global expert id of every slot on rank d (-1 for padding / tail)."""
    epn = cp.E // cp.R
    out = np.full(cp.NvS, -1, dtype=np.int64)
    start = 0
    for g in range(2 * epn):
        e = d * epn + g if g < epn else int(cp.experts_to_copy[d, g - epn])
        cnt = int(cp.alloc[e, d]) if e >= 0 else 0
        out[start:start + cnt] = e
        start = int(cp.cu_seqlens[d, g])
    return out
