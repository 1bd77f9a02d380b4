"""Public API: ``Buffer`` and the collective operations on it.

Interface parity with the reference (moonep/api.py:430-1208):
``Buffer(S, H, K, E, num_ep_ranks, num_sms=None, token_padding=128, group=None,
comm_stream_priority=-1, enable_pdl=True, explicitly_destroy=False)`` with
``dispatch`` / ``prefetch_weight`` / ``combine`` / ``reduce_grad`` (each optionally
``async_finish=True`` on the Buffer's communication stream, returning a CUDA event),
``hidden_nvsh_buffer_view`` / ``router_weight_buffer_view``, ``destroyed`` and ``destroy()``.

Notation: S tokens per rank, K top-k, E routed experts in the EP group, R ranks,
epn = E/R, N = S*K, NvS = dispatched token slots per rank, H hidden size.

What differs underneath: a fresh dispatch is planning (one cross-rank barrier, plan solved
redundantly on every rank) -> dispatch (one exit barrier) -> local duplicate expansion, i.e.
two cross-rank barriers where the reference uses five; the separate pre-sync kernel is only
launched where no later barrier already covers the hazard (plan-reuse dispatch and combine
staging).  Additions: ``check()`` (raises ``MoonEPTimeout`` if a bounded device wait
expired), ``reset()`` (collective re-zeroing of barrier state after such a failure) and
``stats()``.
"""

from __future__ import annotations

import logging
import os
import warnings

import torch
import torch.distributed as dist

from . import engine
from .engine import MoonEPTimeout
from .geometry import Geometry
from .parallel.symm import SymmetricHeap
from .plan import MoonEPCommPlan

logger = logging.getLogger(__name__)
_NVTX = os.environ.get("MOONEP_NVTX", "0") == "1"
_VERIFY_PLANS = os.environ.get("MOONEP_VERIFY_PLANS", "0") == "1"     # debugging: see Buffer.verify_plan
_SLOT_ORDER = os.environ.get("MOONEP_DISPATCH_SLOT_ORDER", "0")       # "0" | "1" | "auto" (4 or more ranks)

PREFETCH_DTYPES = (torch.bfloat16, torch.int8, torch.uint8, torch.float16, torch.float32)


def validate_num_sms(num_sms, max_sms_fn):
    """Type/range validation that must not touch CUDA unless ``num_sms`` is acceptable
    (reference: api.py:231-248)."""
    if num_sms is not None:
        if not isinstance(num_sms, int) or isinstance(num_sms, bool):
            raise TypeError(f"num_sms must be a positive int, got {type(num_sms).__name__}")
        if num_sms <= 0:
            raise ValueError(f"num_sms must be a positive int, got {num_sms}")
    max_sms = max_sms_fn()
    if num_sms is None:
        num_sms = min(32, max_sms)
    if num_sms > max_sms:
        raise ValueError(f"num_sms ({num_sms}) must not exceed the device SM count ({max_sms})")
    return num_sms, max_sms


def num_sms_dedup_from_env(max_sms: int) -> int:
    """``MOONEP_NUM_SMS_DEDUP``: CTA count of the two local duplicate kernels (default all SMs)."""
    raw = os.environ.get("MOONEP_NUM_SMS_DEDUP")
    if raw is None or raw == "":
        return max_sms
    try:
        value = int(raw)
    except ValueError as exc:
        raise ValueError(f"MOONEP_NUM_SMS_DEDUP must be an integer in [1, {max_sms}], got {raw!r}") from exc
    if not (1 <= value <= max_sms):
        raise ValueError(f"MOONEP_NUM_SMS_DEDUP must be in [1, {max_sms}], got {value}")
    return value


def validate_rank_strided_pool(pool: torch.Tensor) -> int:
    """A ``[R, epn, ...]`` view whose rank payloads are contiguous, 16-byte aligned and do not
    overlap; gaps between ranks are allowed (reference: api.py:85-97). Returns the rank stride."""
    assert pool.is_cuda and pool.ndim >= 2 and pool.shape[0] > 0
    assert pool[0].is_contiguous(), "pools must be contiguous within each rank"
    rank_numel = pool[0].numel()
    rank_stride = int(pool.stride(0)) if pool.shape[0] > 1 else max(int(pool.stride(0)), rank_numel)
    assert rank_numel > 0 and rank_stride >= rank_numel, "rank payloads must not overlap"
    stride_bytes = rank_stride * pool.element_size()
    assert stride_bytes % 16 == 0 and 0 < stride_bytes < (1 << 40)
    assert pool.data_ptr() % 16 == 0, "pools must be 16-byte aligned"
    return rank_stride


class TileReady:
    """Handle on the ready flags of one flagged dispatch, handed to the grouped GEMM that consumes
    the dispatched rows (``ops.grouped_gemm.gate_up(..., ready=...)`` / ``dgrad(..., ready=...)``).
    The GEMM then waits tile by tile (128 rows) instead of for the whole dispatch.  ``free_sms`` is
    the number of SMs such a GEMM may occupy while the dispatch kernel is still running."""

    def __init__(self, done_ptr: int, epoch_ptr: int, free_sms: int):
        self.done_ptr, self.epoch_ptr, self.free_sms = done_ptr, epoch_ptr, free_sms


class SlotReady:
    """Handle on the per-slot flags of ``prefetch_weight`` for the grouped GEMM that reads the prefetched
    experts (``ops.grouped_gemm.gate_up(..., slots=...)``): group ``first + b`` of the compute view is
    prefetch slot ``b``; the GEMM waits for a slot's flag before it loads that group's weights."""

    def __init__(self, flags_ptr: int, epoch_ptr: int, first: int):
        self.flags_ptr, self.epoch_ptr, self.first = flags_ptr, epoch_ptr, first


class OpsMixin:
    """The collective operations, written over lists of per-rank arguments.  ``self._states``
    holds the ranks this process hosts (one for ``Buffer``)."""

    _states: list
    geo: Geometry
    _num_sms_dedup: int

    # ---- dispatch with ready flags
    def _dispatch_ready_lists(self, hidden, weights, topk, tpe, plans, comm_stream, *, inter_rank_sync):
        """Planning and the send list on the current stream, then the flagged dispatch kernel on
        ``comm_stream``.  Returns ``(hidden views, weight views, cu_seqlens, plans, event)``; the
        event completes with the dispatch kernel (all rows landed, duplicates expanded)."""
        st, g, n = self._states, self.geo, len(self._states)
        fresh = plans is None
        for i in range(n):
            h = hidden[i]
            assert h.dtype == torch.bfloat16 and h.is_contiguous() and tuple(h.shape) == (g.S, g.H), \
                f"hidden_sh must be a contiguous [S={g.S}, H={g.H}] bf16 tensor"
            if weights is not None:
                w = weights[i]
                assert w.dtype == torch.float32 and w.is_contiguous() and w.numel() == g.N, \
                    "route_weights_sk must be a contiguous [S, K] fp32 tensor"
        cus = [None] * n
        if fresh:
            plans, cus = [], []
            for i in range(n):
                t, c = topk[i].reshape(-1), tpe[i]
                assert t.dtype == torch.int32 and t.numel() == g.N and t.is_contiguous(), \
                    "topk_experts_sk must be a contiguous [S, K] int32 tensor"
                assert c.dtype == torch.int32 and c.numel() == g.E and c.is_contiguous(), \
                    "tokens_per_expert must be a contiguous [E] int32 tensor"
                p, cu = engine.allocate_plan(st[i], with_send_list=True)
                plans.append(p)
                cus.append(cu)
            engine.launch_planning(st, [t.reshape(-1) for t in topk], tpe, plans, cus)
            engine.launch_send_order(st, plans, cus)
        else:
            for p in plans:
                assert isinstance(p, MoonEPCommPlan), "plan must be a MoonEPCommPlan"
                assert (p.N, p.R, p.E, p.NvS, p.K) == (g.N, g.R, g.E, g.NvS, g.K), "plan belongs to another Buffer geometry"
                assert p.send_list is not None, "dispatch_ready needs a plan made by dispatch_ready (it carries the send list)"
        engine.launch_flag_epoch_bump(st)
        main = torch.cuda.current_stream()
        if comm_stream is None or comm_stream == main:
            engine.launch_dispatch(st, hidden, weights, plans, fresh=fresh, entry_barrier=(not fresh) and inter_rank_sync, flagged=True)
            if fresh:
                engine.launch_dup_finalize(st, plans)
            ev = None
        else:
            for t in (*hidden, *(weights or ())):
                t.record_stream(comm_stream)
            comm_stream.wait_event(main.record_event())
            with torch.cuda.stream(comm_stream):
                engine.launch_dispatch(st, hidden, weights, plans, fresh=fresh,
                                       entry_barrier=(not fresh) and inter_rank_sync, flagged=True)
                if fresh:
                    engine.launch_dup_finalize(st, plans)
                ev = comm_stream.record_event()
        out_h = [s.hidden_local for s in st]
        out_w = [s.weights_local if weights is not None else None for s in st]
        return out_h, out_w, cus, plans, ev

    def _slot_ready(self, i: int = 0) -> SlotReady:
        st, g = self._states[i], self.geo
        return SlotReady(st.heap.base + st.rank * st.heap.chunk_bytes + g.off_slotflag, st.scratch["pf_epoch"].data_ptr(), g.epn)

    def _tile_ready(self, i: int = 0) -> TileReady:
        st = self._states[i]
        total = torch.cuda.get_device_properties(st.device).multi_processor_count
        return TileReady(st.scratch["tile_done"].data_ptr(), st.scratch["flag_epoch"].data_ptr(),
                         total - len(self._states) * self.geo.num_sms)

    # ---- dispatch
    def _dispatch_lists(self, hidden, weights, topk, tpe, plans, *, inter_rank_sync, zero_copy, w_zero_copy):
        st = self._states
        g = self.geo
        n = len(st)
        fresh = plans is None
        for i in range(n):
            h = hidden[i]
            assert h.dtype == torch.bfloat16 and h.is_contiguous() and tuple(h.shape) == (g.S, g.H), \
                f"hidden_sh must be a contiguous [S={g.S}, H={g.H}] bf16 tensor"
            if weights is not None:
                w = weights[i]
                assert w.dtype == torch.float32 and w.is_contiguous() and w.numel() == g.N, \
                    "route_weights_sk must be a contiguous [S, K] fp32 tensor"
        cus = [None] * n
        # MOONEP_DISPATCH_SLOT_ORDER=1: the plain call also uses the slot-ordered kernel that expands
        # duplicate rows itself while rows are still arriving (no separate expansion pass)
        slot_order = _SLOT_ORDER == "1" or (_SLOT_ORDER == "auto" and g.R >= 4)
        if fresh:
            plans, cus = [], []
            for i in range(n):
                t, c = topk[i].reshape(-1), tpe[i]
                assert t.dtype == torch.int32 and t.numel() == g.N and t.is_contiguous(), \
                    "topk_experts_sk must be a contiguous [S, K] int32 tensor"
                assert c.dtype == torch.int32 and c.numel() == g.E and c.is_contiguous(), \
                    "tokens_per_expert must be a contiguous [E] int32 tensor"
                p, cu = engine.allocate_plan(st[i], with_send_list=slot_order)
                plans.append(p)
                cus.append(cu)
            engine.launch_planning(st, [t.reshape(-1) for t in topk], tpe, plans, cus)
            if slot_order:
                engine.launch_send_order(st, plans, cus)
        else:
            for p in plans:
                assert isinstance(p, MoonEPCommPlan), "plan must be a MoonEPCommPlan"
                assert (p.N, p.R, p.E, p.NvS, p.K) == (g.N, g.R, g.E, g.NvS, g.K), "plan belongs to another Buffer geometry"
            slot_order = slot_order and all(p.send_list is not None for p in plans)
        # planning's barrier already orders this op after every rank's previous one
        if slot_order:
            engine.launch_flag_epoch_bump(st)
            engine.launch_dispatch(st, hidden, weights, plans, fresh=fresh, entry_barrier=(not fresh) and inter_rank_sync,
                                   flagged=True)
            if fresh:
                engine.launch_dup_finalize(st, plans)
        else:
            engine.launch_dispatch(st, hidden, weights, plans, fresh=fresh,
                                   entry_barrier=(not fresh) and inter_rank_sync)
            pdl = bool(getattr(self, "enable_pdl", False))      # the expansion is scheduled while dispatch drains
            if fresh:
                engine.launch_dup_expand_fresh(st, [s.hidden_local for s in st], plans, self._num_sms_dedup * 4, pdl)
            else:
                engine.launch_dup_expand(st, [s.hidden_local for s in st], plans, self._num_sms_dedup * 4, pdl)
        out_h, out_w = [], []
        for i in range(n):
            if zero_copy:
                out_h.append(st[i].hidden_local)
            else:
                out_h.append(st[i].hidden_local.clone())
            if weights is None:
                out_w.append(None)
            elif w_zero_copy:
                out_w.append(st[i].weights_local)
            else:
                out_w.append(st[i].weights_local.clone())
        return out_h, out_w, cus, plans

    # ---- combine
    def _combine_lists(self, plans, hidden_nvsh, weights_nvs, *, inter_rank_sync, zero_copy, w_zero_copy):
        st = self._states
        g = self.geo
        n = len(st)
        for i in range(n):
            assert isinstance(plans[i], MoonEPCommPlan), "Buffer.combine: plan is required"
            h = hidden_nvsh[i]
            assert h is not None and h.dtype == torch.bfloat16 and h.is_contiguous()
            assert tuple(h.shape) == (g.NvS, g.H), f"hidden_nvsh must be [NvS={g.NvS}, H={g.H}]"
            if weights_nvs is not None and weights_nvs[i] is not None:
                w = weights_nvs[i]
                assert w.dtype == torch.float32 and w.is_contiguous() and tuple(w.shape) == (g.NvS,)
            if zero_copy:
                assert h.data_ptr() == st[i].hidden_local.data_ptr(), (
                    "combine(zero_copy=True): hidden_nvsh must alias the shard view returned by "
                    "dispatch(zero_copy=True)")
            if w_zero_copy and weights_nvs is not None and weights_nvs[i] is not None:
                assert weights_nvs[i].data_ptr() == st[i].weights_local.data_ptr(), (
                    "combine(router_weights_zero_copy=True): route_weights_nvs must alias the weights "
                    "view returned by dispatch(router_weights_zero_copy=True)")
        have_w = weights_nvs is not None and weights_nvs[0] is not None
        staging = (not zero_copy) or (have_w and not w_zero_copy)
        if inter_rank_sync and staging and g.R > 1:
            engine.launch_rank_sync(st)     # peers may still be reading the shard we are about to overwrite
        for i in range(n):
            if not zero_copy:
                st[i].hidden_local.copy_(hidden_nvsh[i])
            if have_w and not w_zero_copy:
                st[i].weights_local.copy_(weights_nvs[i])
        engine.launch_dup_reduce(st, [s.hidden_local for s in st], plans, self._num_sms_dedup * 4)
        outs = [torch.empty(g.S, g.H, dtype=torch.bfloat16, device=s.device) for s in st]
        outw = [torch.empty(g.S, g.K, dtype=torch.float32, device=s.device) for s in st] if have_w else None
        engine.launch_combine(st, plans, outs, outw, entry_barrier=True, pdl=bool(getattr(self, "enable_pdl", False)))
        return outs, outw

    # ---- prefetch / reduce
    def _push_reduce_lists(self, want_weights: bool):
        st, g = self._states, self.geo
        dev = st[0].hidden_local.device
        outs = [torch.empty(g.S, g.H, dtype=torch.bfloat16, device=dev) for _ in st]
        out_ws = [torch.empty(g.S, g.K, dtype=torch.float32, device=dev) for _ in st] if want_weights else None
        engine.launch_push_reduce(st, outs, out_ws, self._num_sms_dedup)
        return outs, out_ws

    def _push_target(self, i: int = 0):
        """``PushTarget`` of rank-state ``i`` for the grouped GEMM's push epilogue."""
        from .ops.grouped_gemm import PushTarget
        st, g = self._states[i], self.geo
        assert g.off_push, "create the Buffer with push_combine=True"
        heap = st.heap
        return PushTarget(st.srcinfo_local, heap.base + g.off_push, heap.base + g.off_pushw, heap.chunk_bytes, g.N, g.R)

    def _check_weight_pairs(self, locals_, pools, dtypes, what):
        g = self.geo
        for local, pool in zip(locals_, pools):
            assert local.dtype in dtypes, f"{what}: unsupported dtype {local.dtype}"
            assert local.is_contiguous()
            assert local.ndim >= 2 and int(local.shape[0]) == g.epn
            assert pool.dtype == local.dtype and validate_rank_strided_pool(pool)
            assert pool.ndim == local.ndim + 1 and tuple(pool.shape[:2]) == (g.R, g.epn)
            assert tuple(pool.shape[2:]) == tuple(local.shape[1:])
            assert pool.device == local.device
            assert (local[0].numel() * local.element_size()) % 16 == 0, f"{what}: expert payload must be a multiple of 16 bytes"
            assert local.data_ptr() % 16 == 0, f"{what}: local tensors must be 16-byte aligned"

    def _prefetch_lists(self, plans, pairs_list, bump_epoch: bool = True):
        engine.launch_prefetch(self._states, [p.experts_to_copy for p in plans], pairs_list, bump_epoch)

    def _reduce_lists(self, plans, pairs_list, inter_rank_sync: bool = True, clear_slots: bool = True):
        engine.launch_grad_reduce(self._states, [p.experts_to_copy for p in plans], pairs_list,
                                  entry_barrier=inter_rank_sync, clear_slots=clear_slots)


class Buffer(OpsMixin):
    """Owner of one rank's communication buffers, scratch and communication stream.

    Must be created after ``torch.distributed.init_process_group`` (any backend: the process
    group only carries handle exchange and barriers at construction / destruction).  Call
    ``destroy()`` before tearing the process group down.
    """

    def __init__(self, S: int, H: int, K: int, E: int, num_ep_ranks: int, num_sms: int | None = None,
                 token_padding: int = 128, group=None, comm_stream_priority: int = -1,
                 enable_pdl: bool = True, explicitly_destroy: bool = False, multicast: bool | None = None,
                 push_combine: bool = False):
        assert isinstance(comm_stream_priority, int), \
            f"comm_stream_priority must be an int, got {type(comm_stream_priority).__name__}"
        assert isinstance(enable_pdl, bool), f"enable_pdl must be a bool, got {type(enable_pdl).__name__}"
        self.explicitly_destroy = explicitly_destroy
        self.comm_stream_priority = comm_stream_priority
        self.enable_pdl = enable_pdl and os.environ.get("MOONEP_PDL", "1") != "0"   # MOONEP_PDL=0: plain launches
        self._destroyed = False
        self._states = []
        self._heap = None
        self._comm_stream = None
        self._group = group
        if multicast is None:      # NVSwitch multicast for the planner's histogram exchange (optional)
            multicast = os.environ.get("MOONEP_MULTICAST", "0") == "1"

        num_sms, max_sms = validate_num_sms(
            num_sms, lambda: torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count)
        R = num_ep_ranks
        if R > 1 or dist.is_initialized():
            rank = dist.get_rank(group=group)
            world = dist.get_world_size(group=group)
        else:
            rank, world = 0, 1
        assert R == world, f"num_ep_ranks ({R}) must equal group world size ({world})"
        self._num_sms_dedup = num_sms_dedup_from_env(max_sms)
        self.geo = Geometry.make(S, H, K, E, R, token_padding, num_sms, push_combine=push_combine)
        device = torch.device("cuda", torch.cuda.current_device())
        if world > 1:
            self._heap = SymmetricHeap.create(self.geo.chunk_bytes, group=group, multicast=multicast)
        else:
            self._heap = SymmetricHeap.local(1, self.geo.chunk_bytes, device)
        self._states = [engine.make_rank_state(self.geo, rank, self._heap, device)]
        self.rank = rank
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier(group=group)
        self._comm_stream = torch.cuda.Stream(device=device, priority=comm_stream_priority)
        if rank == 0:
            g = self.geo
            logger.info("moonep_b200 Buffer: S=%d H=%d K=%d E=%d R=%d NvS=%d num_sms=%d; symmetric chunk %.1f MiB "
                        "(hidden %.1f MiB), heap %.1f MiB mapped", g.S, g.H, g.K, g.E, g.R, g.NvS, g.num_sms,
                        self._heap.chunk_bytes / 2**20, g.NvS * g.H * 2 / 2**20,
                        self._heap.chunk_bytes * world / 2**20)

    # ---- properties
    @property
    def destroyed(self) -> bool:
        return self._destroyed

    def _st(self) -> engine.RankState:
        """Entry check of every public op: the Buffer is alive and no kernel of it has given up a
        wait.  The failure flag is host memory that the kernels write (no synchronisation here), so
        a rank whose peers were late learns of it at its next call instead of computing on with
        unsynchronised data."""
        assert not self._destroyed, "MoonEP Buffer has been destroyed"
        st = self._states[0]
        if engine.failed(st):
            self.check()
        return st

    @property
    def NvS(self) -> int:
        return self.geo.NvS

    @property
    def hidden_nvsh_buffer_view(self) -> torch.Tensor:
        """This rank's ``[NvS, H]`` bf16 communication shard (zero-copy integration). It aliases
        state that every dispatch/combine overwrites: never let autograd save it."""
        return self._st().hidden_local

    @property
    def router_weight_buffer_view(self) -> torch.Tensor:
        """fp32 ``[NvS]`` view of this rank's route-weight slots (same aliasing rules)."""
        return self._st().weights_local

    @property
    def comm_stream(self) -> torch.cuda.Stream:
        return self._comm_stream

    # ---- health
    def check(self) -> None:
        """Synchronise and raise ``MoonEPTimeout`` if any kernel of this Buffer gave up a wait."""
        assert not self._destroyed, "MoonEP Buffer has been destroyed"
        s = engine.read_status(self._states[0])
        if s is not None:
            raise MoonEPTimeout(s)

    def healthy(self) -> bool:
        """False once a kernel of this Buffer has recorded a failure.  Does not synchronise: safe to
        call between launches and between replays of a captured graph (``check()`` gives the details)."""
        return self._destroyed or not engine.failed(self._states[0])

    def reset(self) -> None:
        """Collective: clear barrier words, epochs and the error status after a failed op."""
        assert not self._destroyed, "MoonEP Buffer has been destroyed"
        st = self._states[0]
        torch.cuda.synchronize()
        if self.geo.R > 1:
            dist.barrier(group=self._group)
        g = self.geo
        self._heap.view(st.rank, g.off_bar, (4 * 128,), torch.int32).zero_()
        self._heap.view(st.rank, g.off_ready, (g.ntiles,), torch.int32).zero_()
        self._heap.view(st.rank, g.off_slotflag, (g.epn,), torch.int32).zero_()
        for name in ("grid_bar", "epoch", "send_cnt", "vb_flags", "tile_done", "flag_epoch", "slot_done", "pf_epoch"):
            st.scratch[name].zero_()
        st.status.zero_()
        st.status_host.zero_()
        torch.cuda.synchronize()
        if self.geo.R > 1:
            dist.barrier(group=self._group)

    def stats(self, plan: MoonEPCommPlan) -> dict:
        """Host-side summary of a plan (synchronises): redundancy and duplicate-row counters."""
        rs = plan.remote_stats.tolist()
        dc = plan.dup_counts.tolist()
        zf = plan.zero_fill_ranges[:, 1].sum().item()
        return dict(experts_received=rs[0], slots_sent=rs[1], dup_groups=dc[0], dup_rows=dc[1],
                    dedup_ratio=dc[1] / max(1, plan.N), padded_rows=int(zf))

    def counters(self, reset: bool = False) -> dict:
        """Device-side counters of this Buffer's kernels since creation or the last reset
        (synchronises): dispatch / combine launches, rows sent in total, to other ranks and per
        destination rank, padding rows cleared, rows pulled by combine, duplicate rows expanded by
        flagged dispatches, cross-rank barriers executed and the time spent waiting in them.
        ``MOONEP_COUNTERS=0`` at construction switches the accounting off (empty dict)."""
        return engine.read_counters(self._st(), reset)

    def verify_plan(self, plan: MoonEPCommPlan) -> None:
        """Debugging aid, collective and synchronising: every rank fingerprints its view of the
        plan of one dispatch, the fingerprints are gathered over the process group and compared
        (identical redundant-expert table everywhere, statistics consistent with it, exactly
        ``S*K`` rows arriving on every rank).  Raises ``RuntimeError`` on every rank if the
        replicated planners diverged.  ``MOONEP_VERIFY_PLANS=1`` runs it after every fresh
        synchronous ``dispatch``."""
        from .plan import plan_fingerprint, compare_fingerprints
        self._st()
        fp = plan_fingerprint(plan, self.rank)
        if self.geo.R > 1:
            fps = [None] * self.geo.R
            dist.all_gather_object(fps, fp, group=self._group)
        else:
            fps = [fp]
        errs = compare_fingerprints(fps)
        if errs:
            raise RuntimeError("MoonEP plan check failed: " + "; ".join(errs))

    # ---- async plumbing
    def _run(self, async_finish: bool, tensors, fn, label: str = "moonep.op"):
        nvtx = _NVTX
        if nvtx:            # MOONEP_NVTX=1: one range per public op (visible in Nsight Systems timelines)
            torch.cuda.nvtx.range_push(label + (".async" if async_finish else ""))
        try:
            if not async_finish:
                return fn(), None
            main = torch.cuda.current_stream()
            comm = self._comm_stream
            for t in tensors:
                if isinstance(t, torch.Tensor) and t.is_cuda:
                    t.record_stream(comm)
            comm.wait_event(main.record_event())
            with torch.cuda.stream(comm):
                out = fn()
                done = comm.record_event()
            return out, done
        finally:
            if nvtx:
                torch.cuda.nvtx.range_pop()

    # ---- dispatch
    def dispatch(self, hidden_sh: torch.Tensor, route_weights_sk: torch.Tensor | None = None,
                 topk_experts_sk: torch.Tensor | None = None, tokens_per_expert: torch.Tensor | None = None,
                 plan: MoonEPCommPlan | None = None, async_finish: bool = False, *,
                 inter_rank_sync: bool = True, zero_copy: bool = False, router_weights_zero_copy: bool = False):
        """Run planning (unless ``plan`` is given) and scatter tokens into their expert-grouped
        slots on the destination ranks.

        Returns ``(hidden_nvsh[NvS,H] bf16, route_weights_nvs[NvS] fp32 | None,
        cu_seqlens[2*epn] int32 | None, plan)`` plus a CUDA event when ``async_finish``.
        With a saved ``plan`` (backward of combine) planning is skipped, ``cu_seqlens`` is
        None, the same plan object is returned and its tensors are not modified."""
        self._st()
        if plan is None:
            assert topk_experts_sk is not None and tokens_per_expert is not None, \
                "dispatch needs topk_experts_sk and tokens_per_expert unless a plan is reused"

        def body():
            oh, ow, cus, plans = self._dispatch_lists(
                [hidden_sh], None if route_weights_sk is None else [route_weights_sk],
                None if plan is not None else [topk_experts_sk],
                None if plan is not None else [tokens_per_expert],
                None if plan is None else [plan],
                inter_rank_sync=inter_rank_sync, zero_copy=zero_copy, w_zero_copy=router_weights_zero_copy)
            return oh[0], ow[0], cus[0], plans[0]

        tensors = [hidden_sh, route_weights_sk, topk_experts_sk, tokens_per_expert]
        if plan is not None:
            tensors += list(plan.tensors())
        (h, w, cu, p), ev = self._run(async_finish, tensors, body, "moonep.dispatch")
        if async_finish:
            for t in (h, w, cu, *p.tensors()):
                if isinstance(t, torch.Tensor):
                    t.record_stream(torch.cuda.current_stream())
            return h, w, cu, p, ev
        if plan is None and _VERIFY_PLANS and not torch.cuda.is_current_stream_capturing():
            self.verify_plan(p)
        return h, w, cu, p

    def dispatch_ready(self, hidden_sh: torch.Tensor, route_weights_sk: torch.Tensor | None = None,
                       topk_experts_sk: torch.Tensor | None = None, tokens_per_expert: torch.Tensor | None = None,
                       plan: MoonEPCommPlan | None = None, *, inter_rank_sync: bool = True):
        """``dispatch`` for a consumer that starts before the all-to-all has finished (extension; the
        reference's dispatch ends with a full barrier, moonep/dispatch.py:687-692).

        Planning runs on the current stream, the dispatch kernel on the communication stream.
        Rows are sent in the order of their destination slots, every 128-row tile of the shard gets
        a ready flag, and duplicate rows are expanded by the same kernel as their tile completes.
        Returns ``(hidden_nvsh, route_weights_nvs | None, cu_seqlens | None, plan, ready, event)``:
        the two views are zero-copy and fill up while the kernel runs; ``ready`` (``TileReady``) goes
        to ``ops.grouped_gemm.gate_up`` / ``dgrad`` launched on the current stream with at most
        ``ready.free_sms`` CTAs; anything else that reads the views must wait for ``event``.
        A saved ``plan`` must come from ``dispatch_ready`` (it carries the send list)."""
        self._st()
        if plan is None:
            assert topk_experts_sk is not None and tokens_per_expert is not None, \
                "dispatch needs topk_experts_sk and tokens_per_expert unless a plan is reused"
        if _NVTX:
            torch.cuda.nvtx.range_push("moonep.dispatch_ready")
        try:
            oh, ow, cus, plans, ev = self._dispatch_ready_lists(
                [hidden_sh], None if route_weights_sk is None else [route_weights_sk],
                None if plan is not None else [topk_experts_sk], None if plan is not None else [tokens_per_expert],
                None if plan is None else [plan], self._comm_stream, inter_rank_sync=inter_rank_sync)
        finally:
            if _NVTX:
                torch.cuda.nvtx.range_pop()
        return oh[0], ow[0], cus[0], plans[0], self._tile_ready(0), ev

    # ---- prefetch
    def prefetch_weight(self, plan: MoonEPCommPlan | None = None, async_finish: bool = False, *,
                        local_gate_weight=None, local_up_weight=None, local_down_weight=None,
                        gate_prefetch_buffer=None, up_prefetch_buffer=None, down_prefetch_buffer=None,
                        local_gate_scale=None, local_up_scale=None, local_down_scale=None,
                        gate_scale_prefetch_buffer=None, up_scale_prefetch_buffer=None,
                        down_scale_prefetch_buffer=None):
        """Push this rank's experts that ``plan`` replicated elsewhere into the owners' prefetch
        slots (``*_prefetch_buffer``: ``[R, epn, ...]`` all-rank views; local tensors
        ``[epn, ...]``).  Optional block-scale tensors travel in the same launch."""
        self._st()
        assert isinstance(plan, MoonEPCommPlan), "Buffer.prefetch_weight: plan is required"
        locals_ = (local_gate_weight, local_up_weight, local_down_weight)
        pools = (gate_prefetch_buffer, up_prefetch_buffer, down_prefetch_buffer)
        assert all(t is not None for t in (*locals_, *pools)), "prefetch_weight tensors must be provided together"
        for l in locals_:
            assert l.ndim == 3, "weights must be [epn, rows, cols]"
        self._check_weight_pairs(locals_, pools, PREFETCH_DTYPES, "prefetch_weight")
        pairs = list(zip(locals_, pools))
        scales = (local_gate_scale, local_up_scale, local_down_scale)
        spools = (gate_scale_prefetch_buffer, up_scale_prefetch_buffer, down_scale_prefetch_buffer)
        if any(t is not None for t in (*scales, *spools)):
            assert all(t is not None for t in (*scales, *spools)), "prefetch_weight scales must be provided together"
            self._check_weight_pairs(scales, spools, PREFETCH_DTYPES + (torch.float8_e4m3fn, torch.float8_e8m0fnu)
                                     if hasattr(torch, "float8_e8m0fnu") else PREFETCH_DTYPES, "prefetch_weight scales")
            pairs += list(zip(scales, spools))
        tensors = [plan.experts_to_copy] + [t for pr in pairs for t in pr]
        # the prefetch epoch advances on the CALLER's stream: a GEMM launched there afterwards with
        # slot_ready() reads the new epoch even while the prefetch itself still waits on the comm stream
        engine.launch_pf_epoch_bump(self._states)
        _, ev = self._run(async_finish, tensors, lambda: self._prefetch_lists([plan], [pairs], False), "moonep.prefetch_weight")
        return ev

    def slot_ready(self) -> SlotReady:
        """Per-slot flags of the ``prefetch_weight`` launched last (extension; the reference only has the
        launch's trailing barrier, moonep/prefetch.py:467-470).  Pass it as ``slots=`` to the grouped GEMMs
        that read the compute view ``[local | slots]`` and are launched, in stream order, after that
        ``prefetch_weight`` call was issued (it may still be running on the communication stream): groups of
        prefetched experts are then loaded as soon as their own weights have landed."""
        self._st()
        return self._slot_ready(0)

    # ---- combine
    def combine(self, plan: MoonEPCommPlan | None = None, hidden_nvsh: torch.Tensor | None = None,
                route_weights_nvs: torch.Tensor | None = None, async_finish: bool = False,
                inter_rank_sync: bool = True, *, zero_copy: bool = False, router_weights_zero_copy: bool = False):
        """Sum each token's K rows back to token-major ``[S, H]`` (unweighted; the FFN applies the
        route weights).  Returns ``(hidden_sh, route_weights_sk | None, event | None)``."""
        self._st()

        def body():
            outs, outw = self._combine_lists(
                [plan], [hidden_nvsh], None if route_weights_nvs is None else [route_weights_nvs],
                inter_rank_sync=inter_rank_sync, zero_copy=zero_copy, w_zero_copy=router_weights_zero_copy)
            return outs[0], (outw[0] if outw is not None else None)

        tensors = [hidden_nvsh, route_weights_nvs] + (list(plan.tensors()) if isinstance(plan, MoonEPCommPlan) else [])
        (o, w), ev = self._run(async_finish, tensors, body, "moonep.combine")
        if async_finish:
            for t in (o, w):
                if isinstance(t, torch.Tensor):
                    t.record_stream(torch.cuda.current_stream())
        return o, w, ev

    # ---- push-combine (extension: the reference always pulls)
    def push_target(self):
        """Argument for ``ops.grouped_gemm.down(..., push=...)`` / ``dgrad_gate_up(..., push=...)``:
        with it the GEMM's epilogue stores every output row straight into the receive area of the
        rank the token came from (peer memory), using the provenance table the last ``dispatch``
        of this Buffer wrote.  Needs ``Buffer(..., push_combine=True)``."""
        self._st()
        return self._push_target(0)

    def combine_pushed(self, want_weights: bool = False, async_finish: bool = False):
        """Finish a combine whose rows were pushed by a GEMM epilogue: cross-rank barrier, then the
        local sum over each token's K received rows (ascending k, fp32).  Returns
        ``(hidden_sh [S, H], per-slot scalars [S, K] | None, event | None)``."""
        self._st()
        (o, w), ev = self._run(async_finish, [], lambda: self._push_reduce_lists(want_weights), "moonep.combine_pushed")
        out, ow = o[0], (w[0] if w is not None else None)
        if async_finish:
            for t in (out, ow):
                if isinstance(t, torch.Tensor):
                    t.record_stream(torch.cuda.current_stream())
        return out, ow, ev

    # ---- reduce_grad
    def reduce_grad(self, plan: MoonEPCommPlan | None = None, async_finish: bool = False, *,
                    local_gate_grad=None, local_up_grad=None, local_down_grad=None,
                    gate_reduce_buffer=None, up_reduce_buffer=None, down_reduce_buffer=None,
                    inter_rank_sync: bool = True):
        """Accumulate the gradients of this rank's replicated experts from every rank's reduce
        slots into the local fp32 parameter grads (fixed order), then zero this rank's own
        consumed slots.  The kernel first waits for every rank (``inter_rank_sync``, default on), so
        each holder's reduce-buffer writes queued before its own call are complete when they are read;
        pass ``inter_rank_sync=False`` only if something else already orders the ranks (the reference
        leaves this to the caller, api.py:1154-1158 there)."""
        self._st()
        locals_ = (local_gate_grad, local_up_grad, local_down_grad)
        pools = (gate_reduce_buffer, up_reduce_buffer, down_reduce_buffer)
        assert all(t is not None for t in (*locals_, *pools)), "reduce_grad tensors must be provided together"
        assert isinstance(plan, MoonEPCommPlan), "Buffer.reduce_grad: plan is required"
        for l in locals_:
            assert l.ndim == 3
        self._check_weight_pairs(locals_, pools, (torch.float32,), "reduce_grad")
        pairs = list(zip(locals_, pools))
        tensors = [plan.experts_to_copy] + [t for pr in pairs for t in pr]
        _, ev = self._run(async_finish, tensors, lambda: self._reduce_lists([plan], [pairs], inter_rank_sync), "moonep.reduce_grad")
        return ev

    def reduce_grad_subset(self, plan: MoonEPCommPlan, grads, async_finish: bool = False, *, inter_rank_sync: bool = True,
                           clear_slots: bool = True):
        """``reduce_grad`` for any non-empty subset of the projections: ``grads`` is a sequence of
        ``(local_grad [epn, ...] fp32, reduce_buffer [R, epn, ...] fp32)`` pairs.  Lets a training
        step reduce the gradient of one projection while it still computes the others.  Collective
        like ``reduce_grad``: every rank must issue the same calls in the same order.
        ``clear_slots=False`` leaves the consumed slots as they are (no second barrier, no zeroing): for a
        caller whose next weight-gradient GEMM overwrites every slot it uses.  (Extension: the reference
        only offers the three-projection call.)"""
        self._st()
        assert isinstance(plan, MoonEPCommPlan), "Buffer.reduce_grad_subset: plan is required"
        pairs = [(l, p) for l, p in grads]
        assert 1 <= len(pairs) <= 3, "reduce_grad_subset takes one to three (local_grad, reduce_buffer) pairs"
        self._check_weight_pairs([l for l, _ in pairs], [p for _, p in pairs], (torch.float32,), "reduce_grad_subset")
        tensors = [plan.experts_to_copy] + [t for pr in pairs for t in pr]
        _, ev = self._run(async_finish, tensors, lambda: self._reduce_lists([plan], [pairs], inter_rank_sync, clear_slots),
                          "moonep.reduce_grad")
        return ev

    # ---- teardown
    def destroy(self) -> None:
        """Synchronise and release the symmetric memory. Collective; idempotent."""
        if self._destroyed:
            return
        self._destroyed = True
        try:
            if self._comm_stream is not None:
                self._comm_stream.synchronize()
            torch.cuda.synchronize()
            if self.geo.R > 1 and dist.is_initialized():
                dist.barrier(group=self._group)
        finally:
            for s in self._states:       # drop views before their owner
                s.hidden_local = None
                s.weights_local = None
            self._states = []
            if self._heap is not None:
                self._heap.close()
                self._heap = None

    def __del__(self):
        try:
            if not getattr(self, "_destroyed", True):
                if self.explicitly_destroy:
                    warnings.warn("moonep_b200.Buffer was garbage-collected without destroy()", ResourceWarning)
                else:
                    self.destroy()
        except Exception:
            pass
