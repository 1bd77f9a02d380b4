"""Shared scaffolding of bench_prefetch.py and bench_grad_reduce.py.

Both benchmarks time one collective kernel over expert pools for hand-made redundancy
patterns (which local expert of one owner rank sits in how many peers' spare slots), the
way the reference's benchmarks/bench_prefetch.py:47-110 and bench_grad_reduce.py describe
their cases by a per-expert fan-out list.  Two ways to run:

* under ``torchrun`` with one rank per GPU: real ``Buffer`` + ``ExpertPools`` in symmetric
  memory, traffic crosses NVLink, times are the max over ranks;
* ``--emulate-ranks R`` on one GPU: every rank of the group is hosted by one cooperative
  launch (``sim.LocalCluster``), "peer" memory is another region of the same device, so the
  figure is an HBM number and only useful for regression tracking and profiling.
"""
from __future__ import annotations

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from moonep_b200 import Buffer, MoonEPCommPlan  # noqa: E402
from moonep_b200.pools import ExpertPools, NAMES  # noqa: E402
from moonep_b200.sim.local_cluster import LocalCluster  # noqa: E402

# Buffer geometry is irrelevant to the pool kernels; keep the communication shard tiny.
_S, _H, _K = 8, 128, 2


def cases_for(R: int, H: int, Hp: int):
    """Fan-out patterns for an owner with ``epn`` experts; every count is clamped to R-1."""
    m = max(R - 1, 0)

    def c(label, epn, counts, h=H, hp=Hp):
        return {"label": label, "epn": epn, "H": h, "Hp": hp, "counts": [min(x, m) for x in counts]}

    return [
        c("slots_1", 8, [1, 0, 0, 0, 0, 0, 0, 0]),
        c("slots_3", 8, [2, 1, 0, 0, 0, 0, 0, 0]),
        c("slots_5", 8, [3, 2, 0, 0, 0, 0, 0, 0]),
        c("ramp", 8, [0, 1, 2, 3, 0, 1, 2, 3]),
        c("full", 8, [m] * 8),
        c("epn4_full", 4, [m] * 4),
        c("thin_cols", 8, [3, 0, 2, 1, 3, 0, 2, 1], 7168, 128),
        c("dsv3_expert", 4, [3, 1, 0, 2], 7168, 2048),
    ]


def experts_to_copy_for(R: int, epn: int, owner: int, counts):
    """``[R, epn]`` slot table: local expert ``e`` of ``owner`` is placed on ``counts[e]``
    distinct other ranks (round-robin start so receivers fill evenly), slots ascending."""
    etc = torch.full((R, epn), -1, dtype=torch.int32)
    used = [0] * R
    nxt = 0
    others = [r for r in range(R) if r != owner]
    for e, cnt in enumerate(counts):
        assert cnt <= len(others), "an expert cannot be replicated on more ranks than there are peers"
        for j in range(cnt):
            d = others[(nxt + j) % len(others)]
            assert used[d] < epn
            etc[d, used[d]] = owner * epn + e
            used[d] += 1
        nxt += cnt
    # slots of one rank must list experts in ascending global order (planner contract)
    for d in range(R):
        row = etc[d]
        live = torch.sort(row[row >= 0]).values
        etc[d] = -1
        etc[d, :live.numel()] = live
    return etc


def synthetic_plan(etc: torch.Tensor, NvS: int, K: int, N: int, device) -> MoonEPCommPlan:
    """A plan whose only meaningful field is ``experts_to_copy`` (all the pool kernels read)."""
    R, epn = etc.shape
    z = lambda *s: torch.zeros(*s, dtype=torch.int32, device=device)  # noqa: E731
    return MoonEPCommPlan(dst=z(N), experts_to_copy=etc.to(device).contiguous(), zero_fill_ranges=z(2 * epn, 2),
                          remote_stats=z(2), N=N, R=R, E=R * epn, NvS=NvS, K=K,
                          dup_groups=z(NvS, 3), dup_loffs=z(NvS), dup_counts=z(2))


def time_launches(fn, warmup: int, iters: int, flush: torch.Tensor | None):
    """Median device time in microseconds of ``fn``.  CUDA events on the current stream; the
    launches are queued behind a short device-side sleep without synchronising in between, so
    the host's launch cost (Python argument checks, ~0.1 ms) stays off the device timeline; the
    optional ``flush`` buffer, larger than L2, is rewritten between timed launches."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    torch.cuda._sleep(400_000 * iters)          # ~0.2 ms per queued launch at 1.9 GHz
    for a, b in evs:
        if flush is not None:
            flush.add_(1)
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    ts = sorted(a.elapsed_time(b) * 1e3 for a, b in evs)
    return ts[len(ts) // 2]


class PoolBench:
    """One (R, epn, shapes, dtype) set-up: pools, a buffer or an emulated cluster, and the
    launch callables of the two kernels for a given slot table."""

    def __init__(self, epn: int, H: int, Hp: int, dtype, with_grads: bool, emulate: int, num_sms: int):
        self.epn, self.H, self.Hp, self.dtype = epn, H, Hp, dtype
        self.emulate = emulate
        self.shapes = {"gate": (H, Hp), "up": (H, Hp), "down": (Hp, H)}
        if emulate:
            self.R, self.rank = emulate, 0
            self.dev = torch.device("cuda", torch.cuda.current_device())
            self.cl = LocalCluster(_S, _H, _K, emulate * epn, emulate, num_sms=num_sms, device=str(self.dev))
            self.NvS = self.cl.geo.NvS
            if not with_grads:
                self.w_local = {n: [torch.randn(epn, *self.shapes[n], device=self.dev).to(dtype)
                                    for _ in range(self.R)] for n in NAMES}
                self.w_pool = {n: self.cl.make_pool((epn, *self.shapes[n]), dtype)[0] for n in NAMES}
            else:
                self.g_local = {n: [torch.zeros(epn, *self.shapes[n], device=self.dev) for _ in range(self.R)]
                                for n in NAMES}
                self.g_pool = {n: self.cl.make_pool((epn, *self.shapes[n]), torch.float32)[0] for n in NAMES}
        else:
            self.R = dist.get_world_size() if dist.is_initialized() else 1
            self.rank = dist.get_rank() if dist.is_initialized() else 0
            self.dev = torch.device("cuda", torch.cuda.current_device())
            self.buf = Buffer(_S, _H, _K, self.R * epn, self.R, num_sms=num_sms)
            self.NvS = self.buf.NvS
            self.pools = ExpertPools(epn, *(self.shapes[n] for n in NAMES), dtype=dtype, with_grads=with_grads)
            for n in NAMES:
                w = self.pools.local_weight(n)
                if dtype.is_floating_point:
                    w.normal_()
                else:
                    w.random_(0, 100)

    def plan(self, etc: torch.Tensor) -> MoonEPCommPlan:
        return synthetic_plan(etc, self.NvS, _K, _S * _K, self.dev)

    def prefetch(self, plan):
        if self.emulate:
            pairs = [[(self.w_local[n][r], self.w_pool[n]) for n in NAMES] for r in range(self.R)]
            self.cl.prefetch([plan] * self.R, pairs)
        else:
            self.buf.prefetch_weight(plan, **self.pools.prefetch_kwargs())

    def reduce_grad(self, plan):
        if self.emulate:
            pairs = [[(self.g_local[n][r], self.g_pool[n]) for n in NAMES] for r in range(self.R)]
            self.cl.reduce_grad([plan] * self.R, pairs)
        else:
            self.buf.reduce_grad(plan, **self.pools.reduce_kwargs())

    def check(self):
        (self.cl if self.emulate else self.buf).check()

    def max_over_ranks(self, us: float) -> float:
        if not self.emulate and self.R > 1:
            t = torch.tensor([us], device=self.dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t)
        return us

    def close(self):
        torch.cuda.synchronize()
        if not self.emulate:
            self.pools.destroy()
            self.buf.destroy()
        else:
            for name in ("w_local", "w_pool", "g_local", "g_pool"):
                self.__dict__.pop(name, None)
            self.cl.heap.close()
            self.cl = None
            torch.cuda.empty_cache()


def init_dist():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl")
    return world, int(os.environ.get("RANK", "0"))
