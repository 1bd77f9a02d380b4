"""Per-rank device state and thin launch wrappers around the native kernels.

Every wrapper takes LISTS (one entry per rank hosted by this process): a normal
``Buffer`` passes lists of length one; the single-GPU ``LocalCluster`` passes all R ranks
so that one cooperative launch runs every rank's CTAs side by side (blockIdx.y = rank)
and the cross-rank barriers work on one device.
"""

from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass, field

import torch

from . import _native
from ._native import (MepRankCtx, PlanArgs, DispatchArgs, DupFinalizeArgs, DupArgs, CombineArgs, PushReduceArgs,
                      PrefetchArgs, GradReduceArgs, SendOrderArgs, ptr)
from .geometry import Geometry
from .plan import MoonEPCommPlan

ERROR_NAMES = {1: "grid barrier timed out (a CTA never arrived)",
               2: "cross-rank barrier timed out (a peer never arrived)",
               3: "index out of range",
               4: "ready flag never reached its expected value",
               5: "mbarrier phase never completed"}
KERNEL_NAMES = {1: "rank_sync", 2: "planning", 3: "dispatch", 4: "dup_expand", 5: "dup_reduce", 6: "combine",
                7: "prefetch", 8: "grad_reduce", 9: "grouped_gemm", 10: "wait_probe"}


class MoonEPTimeout(RuntimeError):
    """A bounded device-side wait expired (or a checked index was out of range)."""

    def __init__(self, status: dict):
        self.status = status
        super().__init__(
            f"rank {status['rank']}: {KERNEL_NAMES.get(status['kernel'], status['kernel'])} kernel, site "
            f"{status['site']}: {ERROR_NAMES.get(status['code'], status['code'])} "
            f"(peer/cta {status['peer']}, observed {status['observed']}, expected {status['expected']})")


def wait_budget_ns() -> int:
    ms = float(os.environ.get("MOONEP_WAIT_BUDGET_MS", "2000"))
    return max(1, int(ms * 1e6))


@dataclass
class RankState:
    geo: Geometry
    rank: int
    heap: object
    device: torch.device
    ctx_host: MepRankCtx = None
    ctx_dev: torch.Tensor = None
    scratch: dict = field(default_factory=dict)
    hidden_local: torch.Tensor = None     # [NvS, H] bf16 view of this rank's shard
    weights_local: torch.Tensor = None    # [NvS] fp32 view
    srcinfo_local: torch.Tensor = None    # [NvS] int32 provenance table (push-combine Buffers only)
    status: torch.Tensor = None           # int32[8] device
    status_host: torch.Tensor = None      # int32[1] pinned host memory the kernels mirror status[0] into
    plan_fast: bool = False

    @property
    def ctx_ptr(self) -> int:
        return self.ctx_dev.data_ptr()


def make_rank_state(geo: Geometry, rank: int, heap, device, budget_ns: int | None = None) -> RankState:
    dev = torch.device(device)
    st = RankState(geo, rank, heap, dev)
    i32 = dict(dtype=torch.int32, device=dev)
    R, E, epn = geo.R, geo.E, geo.epn
    s = st.scratch
    s["grid_bar"] = torch.zeros(4, **i32)
    s["epoch"] = torch.zeros(_native.BAR_ROWS, **i32)
    s["hist"] = torch.zeros(geo.num_vblocks * E, **i32)
    s["vb_flags"] = torch.zeros(geo.num_vblocks + 2, **i32)      # + the fast planner's epoch word and exit counter
    s["count"] = torch.zeros(E, **i32)
    s["tpe_prefix"] = torch.zeros(E, **i32)
    s["remaining"] = torch.zeros(E, **i32)
    s["alloc"] = torch.zeros(E * R, **i32)
    s["alloc_cumsum"] = torch.zeros(E * R, **i32)
    s["expert_off"] = torch.zeros(R * E, **i32)
    s["etc_all"] = torch.zeros(R * epn, **i32)
    s["stats_all"] = torch.zeros(R * 2, **i32)
    s["send_cnt"] = torch.zeros(2 * R, dtype=torch.int64, device=dev)     # two halves, see planning_fast_kernel
    s["tile_done"] = torch.zeros(geo.ntiles, **i32)           # ready flags: epoch at which a tile became complete
    s["flag_epoch"] = torch.zeros(4, **i32)                   # [0] flagged dispatches issued, [1] expander ticket
    s["slot_done"] = torch.zeros(R * epn, **i32)              # prefetch: chunks finished per (rank, slot), self-resetting
    s["pf_epoch"] = torch.zeros(2, **i32)                     # prefetch launches issued
    if os.environ.get("MOONEP_COUNTERS", "1") != "0":
        s["counters"] = torch.zeros(_native.COUNTER_SLOTS, dtype=torch.int64, device=dev)
    st.status = torch.zeros(8, **i32)
    # first failure code, mirrored by the kernels into host memory the device can write: the host
    # tests it without synchronising (see Buffer._st)
    st.status_host = torch.zeros(1, dtype=torch.int32).pin_memory()

    c = MepRankCtx()
    c.rank, c.R, c.S, c.H, c.K, c.E, c.epn, c.N, c.NvS = rank, R, geo.S, geo.H, geo.K, E, epn, geo.N, geo.NvS
    c.token_padding, c.vblock_entries, c.num_vblocks = geo.token_padding, geo.vblock_entries, geo.num_vblocks
    c.num_sms = geo.num_sms
    c.checked = 1 if os.environ.get("MOONEP_CHECKED") == "1" else 0
    c.heap_base, c.chunk_stride = heap.base, heap.chunk_bytes
    for name in ("off_hidden", "off_weights", "off_tpe", "off_bar", "off_dupcnt", "off_dupgroups",
                 "off_duploffs", "off_ready", "off_rowsrc", "off_slotflag"):
        setattr(c, name, getattr(geo, name))
    c.dup_group_cap, c.dup_loff_cap = geo.dup_group_cap, geo.dup_loff_cap
    for name in ("grid_bar", "epoch", "hist", "count", "tpe_prefix", "remaining", "alloc", "alloc_cumsum",
                 "expert_off", "etc_all", "stats_all", "send_cnt", "vb_flags", "tile_done", "flag_epoch", "slot_done",
                 "pf_epoch"):
        setattr(c, name, s[name].data_ptr())
    c.ntiles = geo.ntiles
    c.counters = s["counters"].data_ptr() if "counters" in s else None
    c.status = st.status.data_ptr()
    c.status_host = st.status_host.data_ptr()
    c.wait_budget_ns = wait_budget_ns() if budget_ns is None else budget_ns
    c.mc_base = getattr(heap, "mc_base", 0) or None
    if os.environ.get("MOONEP_TRACE") == "1":
        cap = int(os.environ.get("MOONEP_TRACE_RECORDS", "65536"))
        s["trace"] = torch.zeros(1 + 2 * cap, dtype=torch.int64, device=dev)
        c.trace, c.trace_cap = s["trace"].data_ptr(), cap
    st.ctx_host = c
    raw = bytes(c)
    st.ctx_dev = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(dev)
    st.plan_fast = bool(_native.load().mep_planning_is_fast(E, R))
    st.hidden_local = heap.view(rank, geo.off_hidden, (geo.NvS, geo.H), torch.bfloat16)
    st.weights_local = heap.view(rank, geo.off_weights, (geo.NvS,), torch.float32)
    st.srcinfo_local = heap.view(rank, geo.off_srcinfo, (geo.NvS,), torch.int32) if geo.off_srcinfo else None
    return st


def failed(st: RankState) -> bool:
    """True once any kernel of this rank has recorded a failure. A plain read of host memory: no
    synchronisation, usable between launches and during CUDA-graph replays."""
    return int(st.status_host[0]) != 0


def read_counters(st: RankState, reset: bool = False) -> dict:
    """Per-op device counters accumulated since the Buffer was created or last reset (synchronises)."""
    t = st.scratch.get("counters")
    if t is None:
        return {}
    v = t.cpu().tolist()
    out = {name: int(v[i]) for i, name in _native.COUNTER_NAMES.items()}
    out["rows_sent_to"] = [int(x) for x in v[_native.COUNTER_PEER_BASE:_native.COUNTER_PEER_BASE + min(st.geo.R, 48)]]
    if reset:
        t.zero_()
    return out


def read_status(st: RankState) -> dict | None:
    v = st.status.cpu().tolist()
    if v[0] == 0:
        return None
    return dict(code=v[0], kernel=v[1], site=v[2], rank=v[3], peer=v[4],
                observed=v[5] & 0xFFFFFFFF, expected=v[6] & 0xFFFFFFFF)


def read_trace(st: RankState, reset: bool = True):
    """Device timestamps recorded since the last reset: list of ``(ns, kernel, site, cta, warp)``
    sorted by time (needs ``MOONEP_TRACE=1`` when the Buffer was created). Synchronises."""
    t = st.scratch.get("trace")
    if t is None:
        return []
    v = t.cpu()
    n = min(int(v[0]), (v.numel() - 1) // 2)
    out = []
    for i in range(n):
        ns, tag = int(v[1 + 2 * i]), int(v[2 + 2 * i])
        out.append((ns, (tag >> 48) & 0xFFFF, (tag >> 32) & 0xFFFF, (tag >> 8) & 0xFFFFFF, tag & 0xFF))
    if reset:
        t[0] = 0
    return sorted(out)


def _pack(states):
    return _native.ctx_array([s.ctx_ptr for s in states])


def allocate_plan(st: RankState, with_send_list: bool = False):
    """Plan-owned tensors plus cu_seqlens for one rank (reference: planning.py:1168-1215)."""
    g = st.geo
    i32 = dict(dtype=torch.int32, device=st.device)
    extra = dict(send_list=torch.empty(g.N, **i32), send_meta=torch.zeros(4, **i32)) if with_send_list else {}
    plan = MoonEPCommPlan(
        dst=torch.empty(g.N, **i32),
        experts_to_copy=torch.empty(g.R, g.epn, **i32),
        zero_fill_ranges=torch.empty(2 * g.epn, 2, **i32),
        remote_stats=torch.empty(2, **i32),
        N=g.N, R=g.R, E=g.E, NvS=g.NvS, K=g.K,
        dup_groups=torch.empty(g.NvS, 3, **i32),
        dup_loffs=torch.empty(g.NvS, **i32),
        dup_counts=torch.zeros(2, **i32),
        **extra,
    )
    cu = torch.empty(2 * g.epn, **i32)
    return plan, cu


def launch_planning(states, topk_list, tpe_list, plans, cu_list):
    lib = _native.load()
    n = len(states)
    args = (PlanArgs * n)()
    for i in range(n):
        p = plans[i]
        st = states[i]
        args[i] = PlanArgs(ptr(topk_list[i]), ptr(tpe_list[i]), ptr(p.dst), ptr(cu_list[i]),
                           ptr(p.experts_to_copy), ptr(p.zero_fill_ranges), ptr(p.remote_stats),
                           1 if st.plan_fast else 0, 0)
    g = states[0].geo
    _native.check(lib.mep_launch_planning(n, _pack(states), args, g.num_sms, g.E, g.R, _native.cur_stream()), "planning")


def launch_dispatch(states, hidden_list, weights_list, plans, fresh: bool, entry_barrier: bool, flagged: bool = False):
    lib = _native.load()
    n = len(states)
    g0 = states[0].geo
    args = (DispatchArgs * n)()
    for i in range(n):
        w = weights_list[i] if weights_list is not None else None
        fresh_code = 3 if states[i].plan_fast else 1      # which send_cnt half the planner used (3: device epoch)
        args[i] = DispatchArgs(ptr(hidden_list[i]), ptr(w), ptr(plans[i].dst), ptr(plans[i].zero_fill_ranges),
                               fresh_code if fresh else 0, 1 if entry_barrier else 0, g0.off_srcinfo,
                               ptr(plans[i].send_list), ptr(plans[i].send_meta))
    g = states[0].geo
    fn = lib.mep_launch_dispatch_flagged if flagged else lib.mep_launch_dispatch
    _native.check(fn(n, _pack(states), args, g.num_sms, g.H, g.epn, _native.cur_stream()), "dispatch")


def launch_send_order(states, plans, cu_list):
    """Build each plan's send list (``plan.send_list`` / ``plan.send_meta``) from ``plan.dst``."""
    lib = _native.load()
    n = len(states)
    args = (SendOrderArgs * n)()
    g = states[0].geo
    for i in range(n):
        sc = states[i].scratch
        if "send_hist" not in sc:       # bucket histogram and per-entry bucket, sized on first use
            nb = lib.mep_send_order_buckets(g.NvS, g.R, None)
            sc["send_hist"] = torch.zeros(nb, dtype=torch.int32, device=states[i].device)
            sc["send_bucket"] = torch.empty(g.N, dtype=torch.int32, device=states[i].device)
        args[i] = SendOrderArgs(ptr(plans[i].dst), ptr(cu_list[i]), ptr(plans[i].send_list), ptr(plans[i].send_meta),
                                ptr(sc["send_hist"]), ptr(sc["send_bucket"]))
    _native.check(lib.mep_launch_send_order(n, _pack(states), args, g.N, g.NvS, g.R, _native.cur_stream()), "send_order")


def launch_flag_epoch_bump(states):
    """A flagged dispatch is about to be issued: advance the flag epoch on the current stream, ahead
    of the dispatch kernel and of every consumer of its tile flags."""
    lib = _native.load()
    _native.check(lib.mep_launch_flag_epoch_bump(len(states), _pack(states), _native.cur_stream()), "flag_epoch_bump")


def launch_tile_wait_probe(st: RankState, tile: int):
    lib = _native.load()
    _native.check(lib.mep_launch_tile_wait_probe(C.c_void_p(st.ctx_ptr), tile, _native.cur_stream()), "tile_wait_probe")


def launch_dup_finalize(states, plans):
    lib = _native.load()
    n = len(states)
    args = (DupFinalizeArgs * n)()
    for i in range(n):
        args[i] = DupFinalizeArgs(ptr(plans[i].dup_groups), ptr(plans[i].dup_loffs), ptr(plans[i].dup_counts))
    _native.check(lib.mep_launch_dup_finalize(n, _pack(states), args, _native.cur_stream()), "dup_finalize")


def launch_dup_expand_fresh(states, bufs, plans, num_blocks: int, pdl: bool = False):
    """Fresh dispatch: compact the staged duplicate groups into the plan and expand them, one launch.
    ``pdl``: programmatic dependent launch behind the kernel queued just before on this stream."""
    lib = _native.load()
    _native.check(lib.mep_launch_dup_expand_fresh(len(states), _pack(states), _dup_args(states, bufs, plans),
                                                  num_blocks, 1 if pdl else 0, _native.cur_stream()), "dup_expand_fresh")


def _dup_args(states, bufs, plans):
    n = len(states)
    args = (DupArgs * n)()
    for i in range(n):
        args[i] = DupArgs(ptr(bufs[i]), ptr(plans[i].dup_groups), ptr(plans[i].dup_loffs), ptr(plans[i].dup_counts))
    return args


def _dup_check(states, bufs, plans, num_blocks: int, kernel_id: int):
    """MOONEP_CHECKED=1: validate the duplicate tables in a pass of their own before they are used."""
    if states[0].ctx_host.checked:
        lib = _native.load()
        _native.check(lib.mep_launch_dup_check(len(states), _pack(states), _dup_args(states, bufs, plans), num_blocks,
                                               kernel_id, _native.cur_stream()), "dup_check")


def launch_dup_expand(states, bufs, plans, num_blocks: int, pdl: bool = False):
    lib = _native.load()
    _dup_check(states, bufs, plans, num_blocks, 4)
    pdl = pdl and not states[0].ctx_host.checked        # the check sits between dispatch and this kernel
    _native.check(lib.mep_launch_dup_expand(len(states), _pack(states), _dup_args(states, bufs, plans),
                                            num_blocks, 1 if pdl else 0, _native.cur_stream()), "dup_expand")


def launch_dup_reduce(states, bufs, plans, num_blocks: int):
    lib = _native.load()
    _dup_check(states, bufs, plans, num_blocks, 5)
    _native.check(lib.mep_launch_dup_reduce(len(states), _pack(states), _dup_args(states, bufs, plans),
                                            num_blocks, _native.cur_stream()), "dup_reduce")


def launch_combine(states, plans, outs, out_weights, entry_barrier: bool = True, pdl: bool = False):
    lib = _native.load()
    n = len(states)
    args = (CombineArgs * n)()
    for i in range(n):
        ow = out_weights[i] if out_weights is not None else None
        args[i] = CombineArgs(ptr(plans[i].dst), ptr(outs[i]), ptr(ow), 1 if entry_barrier else 0)
    _native.check(lib.mep_launch_combine(n, _pack(states), args, states[0].geo.num_sms, 1 if pdl else 0, _native.cur_stream()), "combine")


def launch_rank_sync(states):
    lib = _native.load()
    _native.check(lib.mep_launch_rank_sync(len(states), _pack(states), _native.cur_stream()), "rank_sync")


def _rank_stride_bytes(pool: torch.Tensor) -> int:
    return int(pool.stride(0)) * pool.element_size()


def launch_pf_epoch_bump(states):
    """A prefetch is about to be issued: advance the prefetch epoch.  Must run in stream order before the
    prefetch kernel AND before any GEMM that waits on its slot flags, i.e. on the stream both are forked from."""
    lib = _native.load()
    _native.check(lib.mep_launch_pf_epoch_bump(len(states), _pack(states), _native.cur_stream()), "pf_epoch_bump")


def launch_prefetch(states, etc_list, tensor_pairs_list, bump_epoch: bool = True):
    """``tensor_pairs_list[i]`` = sequence of up to six ``(local[epn,...], pool[R,epn,...])``.
    ``bump_epoch=False``: the caller has already advanced the prefetch epoch (``launch_pf_epoch_bump``)."""
    lib = _native.load()
    n = len(states)
    args = (PrefetchArgs * n)()
    for i in range(n):
        a = PrefetchArgs()
        a.etc = ptr(etc_list[i])
        pairs = tensor_pairs_list[i]
        a.ntensors = len(pairs)
        for j, (local, pool) in enumerate(pairs):
            a.t[j].local = local.data_ptr()
            a.t[j].pool = pool.data_ptr()
            a.t[j].expert_bytes = local[0].numel() * local.element_size()
            a.t[j].rank_stride = _rank_stride_bytes(pool)
        args[i] = a
    g = states[0].geo
    # new prefetch epoch first (stream order): the kernel stamps completed slots with it and a GEMM that
    # consumes the slots while the prefetch runs compares against it
    if bump_epoch:
        launch_pf_epoch_bump(states)
    _native.check(lib.mep_launch_prefetch(n, _pack(states), args, g.num_sms, g.R, g.epn, _native.cur_stream()), "prefetch")


def launch_grad_reduce(states, etc_list, tensor_pairs_list, entry_barrier: bool = True, clear_slots: bool = True):
    """``entry_barrier``: wait for every rank before the first peer read (the holders' weight-gradient
    GEMMs are then complete).  ``clear_slots=False`` skips the second barrier and the zeroing of the
    consumed slots (for callers that overwrite, not accumulate into, the slots they use next time)."""
    lib = _native.load()
    n = len(states)
    args = (GradReduceArgs * n)()
    for i in range(n):
        a = GradReduceArgs()
        a.etc = ptr(etc_list[i])
        a.flags = (1 if entry_barrier else 0) | (4 if clear_slots else 2)
        pairs = tensor_pairs_list[i]
        a.ntensors = len(pairs)
        for j, (local, pool) in enumerate(pairs):
            a.t[j].local = local.data_ptr()
            a.t[j].pool = pool.data_ptr()
            a.t[j].expert_elems = local[0].numel()
            a.t[j].rank_stride = _rank_stride_bytes(pool)
        args[i] = a
    g = states[0].geo
    _native.check(lib.mep_launch_grad_reduce(n, _pack(states), args, g.num_sms, g.R, g.epn, _native.cur_stream()), "grad_reduce")
    if clear_slots:     # behind the kernel's second barrier, on all SMs (the cooperative kernel's few CTAs store slowly)
        sms = torch.cuda.get_device_properties(states[0].device).multi_processor_count
        _native.check(lib.mep_launch_grad_clear(n, _pack(states), args, 2 * sms, _native.cur_stream()), "grad_clear")


def launch_push_reduce(states, outs, out_ws, num_blocks):
    """Entry barrier + local sum over k of the rows the GEMM epilogues pushed into each rank's
    receive area (push-combine)."""
    lib = _native.load()
    n = len(states)
    args = (PushReduceArgs * n)()
    g = states[0].geo
    assert g.off_push, "this Buffer was created without the push-combine regions"
    for i in range(n):
        args[i] = PushReduceArgs(ptr(outs[i]), ptr(out_ws[i]) if out_ws is not None else None, g.off_push, g.off_pushw)
    _native.check(lib.mep_launch_push_reduce(n, _pack(states), args, num_blocks, _native.cur_stream()), "push_reduce")


def launch_wait_probe(st: RankState, flag: torch.Tensor, expected: int):
    lib = _native.load()
    _native.check(lib.mep_launch_wait_probe(C.c_void_p(st.ctx_ptr), C.c_void_p(flag.data_ptr()),
                                            C.c_uint32(expected), _native.cur_stream()), "wait_probe")
