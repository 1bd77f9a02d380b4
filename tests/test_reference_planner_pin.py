"""Pins this package's planner oracle (``moonep_b200.sim.planner``) to the reference's own executable
specification, ``tests/planning_reference.py`` of the reference checkout, run unmodified in this
process.  Skipped when no reference checkout is found (``MOONEP_REFERENCE_DIR``, or a directory
``reference`` beside this repository).

* allocation table ``alloc[R, E]`` (its ``return_alloc=True`` path needs no process group) on
  many random and skewed routings at R = 2, 4, 8;
* every table -- ``dst`` with its duplicate sign encoding, ``cu_seqlens``, ``experts_to_copy``,
  ``remote_stats``, ``zero_fill_ranges`` and the duplicate groups (as sets) -- at R = 1, 2, 4, 8.  The
  reference gathers all ranks' ``dst`` with ``dist.all_gather``; here that one call is served from a
  table filled by a first pass over the ranks, so no process group is needed.
"""
import importlib.util
import os
from pathlib import Path

import numpy as np
import pytest
import torch

from moonep_b200 import routing
from moonep_b200.geometry import Geometry
from moonep_b200.sim import plan_cluster, dup_table_from_arrays


def _load_reference():
    root = Path(__file__).resolve().parent.parent
    cands = [os.environ.get("MOONEP_REFERENCE_DIR"), root.parent / "reference"]
    for c in cands:
        if c and (Path(c) / "tests" / "planning_reference.py").exists():
            spec = importlib.util.spec_from_file_location("_ref_planning", Path(c) / "tests" / "planning_reference.py")
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            return mod
    return None


REF = _load_reference()
pytestmark = pytest.mark.skipif(REF is None, reason="no reference checkout with tests/planning_reference.py")


def _routing(kind, S, K, E, R, seed):
    if kind == "uniform":
        g = torch.Generator().manual_seed(seed)
        return [torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(S)]).to(torch.int32) for _ in range(R)]
    sigma = {"mild": 0.5, "skewed": 1.5, "extreme": 4.0}[kind]
    return [routing.lognormal_topk(S, K, E, R, sigma, seed, r)[0] for r in range(R)]


def _ctx(rank, S, K, E, R, pad):
    geo = Geometry.make(S, 8, K, E, R, pad, 1)
    return {"rank": rank, "R": R, "E": E, "S": S, "K": K, "NvS_capacity": S * K, "NvS": geo.NvS, "token_padding": pad}, geo


ALLOC_CASES = [(R, kind, seed) for R in (2, 4, 8) for kind in ("uniform", "mild", "skewed", "extreme") for seed in range(10)]


@pytest.mark.parametrize("R,kind,seed", ALLOC_CASES, ids=[f"R{r}-{k}-{s}" for r, k, s in ALLOC_CASES])
def test_allocation_table_equals_the_reference(R, kind, seed):
    S, K, epn = 96, 4, 3 + seed % 4
    E = R * epn
    topk = _routing(kind, S, K, E, R, 100 + seed)
    tpe = torch.stack([torch.bincount(t.flatten().long(), minlength=E).to(torch.int32) for t in topk])
    ctx, _ = _ctx(0, S, K, E, R, 16)
    want = REF.launch_planning_torch_reference(ctx, torch.stack(topk), tpe, return_alloc=True)      # [R, E]
    cp = plan_cluster(np.stack([t.numpy() for t in topk]), E, 16)
    assert np.array_equal(cp.alloc.T, want.numpy()), "alloc differs from the reference planner"


class _Gather:
    """Stands in for ``torch.distributed`` inside the reference module: ``all_gather`` of the ranks'
    ``dst`` is answered from ``table`` (the caller's own tensor for its own rank)."""

    def __init__(self, rank, table):
        self.rank, self.table = rank, table

    def all_gather(self, out, mine, group=None):
        for i, o in enumerate(out):
            o.copy_(mine if i == self.rank else self.table[i])


FULL_CASES = [(1, "skewed", 16, 0), (1, "uniform", 1, 1), (2, "skewed", 16, 2), (2, "extreme", 8, 3), (4, "mild", 32, 4),
              (4, "extreme", 16, 5), (8, "skewed", 16, 6), (8, "uniform", 128, 7)]


@pytest.mark.parametrize("R,kind,pad,seed", FULL_CASES, ids=[f"R{r}-{k}-pad{p}" for r, k, p, _ in FULL_CASES])
def test_every_plan_table_equals_the_reference(R, kind, pad, seed, monkeypatch):
    S, K, epn = 40, 4, 5
    E = R * epn
    topk = _routing(kind, S, K, E, R, 7 + seed)
    tpe = torch.stack([torch.bincount(t.flatten().long(), minlength=E).to(torch.int32) for t in topk])
    cp = plan_cluster(np.stack([t.numpy() for t in topk]), E, pad)
    N = S * K
    # pass 0 placeholder for the other ranks' dst: spread every token's entries over the ranks, so that
    # the reference's duplicate tables (sized NvS) cannot overflow before the real values are known
    idx = torch.arange(N)
    table = [(((idx % K) % R) * cp.NvS + idx // K).to(torch.int32) for _ in range(R)]
    results = None
    for _pass in range(2):          # pass 0 collects every rank's dst, pass 1 sees all of them
        results = []
        for r in range(R):
            ctx, geo = _ctx(r, S, K, E, R, pad)
            assert geo.NvS == cp.NvS
            monkeypatch.setattr(REF, "dist", _Gather(r, table))
            results.append(REF.launch_planning_torch_reference(ctx, torch.stack(topk), tpe))
        for r in range(R):
            d = results[r][0]
            table[r] = torch.where(d >= 0, d, -d - 1).to(torch.int32)
    for r in range(R):
        dst, cu, etc, stats, zfr, dedup = results[r]
        assert np.array_equal(dst.numpy(), cp.dst[r]), f"rank {r}: dst"
        assert np.array_equal(cu.numpy(), cp.cu_seqlens[r]), f"rank {r}: cu_seqlens"
        assert np.array_equal(etc.numpy(), cp.experts_to_copy), f"rank {r}: experts_to_copy"
        assert np.array_equal(stats.numpy(), cp.remote_stats[r]), f"rank {r}: remote_stats"
        assert np.array_equal(zfr.numpy(), cp.zero_fill_ranges[r]), f"rank {r}: zero_fill_ranges"
        got = dup_table_from_arrays(dedup.dup_groups.numpy(), dedup.dup_loffs.numpy(), dedup.dup_counts.numpy())
        want = {k: tuple(sorted(v)) for k, v in cp.dup_tables[r].items()}
        assert got == want, f"rank {r}: duplicate groups"
