"""Expert-parallel MoE FFN built on ``Buffer`` + the tcgen05 grouped GEMM.

Forward  : dispatch -> [prefetch_weight on the comm stream] -> gate/up GEMM with fused
           SwiGLU and route-weight scaling (local experts first, prefetched experts once their
           weights have landed; the private copy of the dispatched tokens that the backward
           pass needs is taken on a side stream meanwhile) -> down GEMM writing straight into
           the communication shard -> combine (zero copy).
           With ``ready_flags`` (default) the dispatch kernel runs on the comm stream and publishes
           a flag per 128-row tile; the gate/up GEMM of the local experts starts at once on the SMs
           that kernel leaves free and takes each tile as it completes, and a second launch of the
           same GEMM (same ticket counter) joins on the comm stream once dispatch and prefetch have
           given their SMs back.
Backward : re-dispatch of the output grad with the saved plan (flagged in the same way, feeding
           dgrad(down)) -> dgrad(down) -> SwiGLU backward
           (also yields the route-weight grads) -> wgrad(down), wgrad(gate) -> [reduce_grad of
           those two on the comm stream] beside dgrad(gate/up) into the shard -> [combine with
           the route-weight-grad channel on the comm stream] beside wgrad(up) -> reduce_grad(up).
           An optional per-projection hook lets the optimizer update a projection as soon as its
           gradient is final, beside the remaining GEMMs.
This is the integration the reference leaves to the training framework (README.md:110-156 of
the reference gives the same operator mapping).  Weights are ``[2*epn, in, out]`` compute views
of an ``ExpertPools``; weight grads are fp32 ``[2*epn, in, out]`` whose tail is the reduce slots.
"""

from __future__ import annotations

import os
from dataclasses import dataclass

import torch

from .api import Buffer
from .ops import grouped_gemm as gg
from .plan import MoonEPCommPlan
from .pools import ExpertPools


@dataclass
class MoEContext:
    plan: MoonEPCommPlan
    cu: torch.Tensor
    x: torch.Tensor          # dispatched tokens [NvS, H] (own copy)
    w_nvs: torch.Tensor      # route weight per slot [NvS]
    act: torch.Tensor        # weighted activation [NvS, H']
    gu: torch.Tensor         # pre-activations [NvS, 2H']


_DEFERRED: list = []       # layers whose last gradient reduction is still running (see wait_grads)


def update_mask(experts_to_copy, rank: int, epn: int, mask=None, hit=None, ones=None):
    """int32 ``[2*epn]`` over the groups of the compute view ``[local | slots]``: 1 for the local experts whose
    gradient is complete on this rank (``experts_to_copy`` -- ``[R, epn]``, expert id held by every slot of every
    rank, -1 for none -- names no replica of them), 0 for replicated local experts and for the slots.
    Pure tensor ops on the table's device, no host synchronisation; ``mask`` / ``hit`` / ``ones`` are optional
    preallocated work tensors (``[2*epn]``, ``[epn+1]``, ``[R*epn]`` int32)."""
    dev = experts_to_copy.device
    flat = experts_to_copy.reshape(-1)
    if mask is None:
        mask = torch.zeros(2 * epn, dtype=torch.int32, device=dev)
    if hit is None:
        hit = torch.zeros(epn + 1, dtype=torch.int32, device=dev)
    if ones is None:
        ones = torch.ones(flat.numel(), dtype=torch.int32, device=dev)
    idx = flat.long() - rank * epn
    idx = torch.where((idx >= 0) & (idx < epn), idx, torch.full_like(idx, epn))
    hit.zero_()
    hit.scatter_(0, idx, ones)
    mask[:epn] = 1 - hit[:epn]
    mask[epn:] = 0
    return mask


class ExpertParallelMoE:
    def __init__(self, buffer: Buffer, pools: ExpertPools, overlap_prefetch: bool = True,
                 overlap_backward: bool | None = None, ready_flags: bool | None = None):
        g = buffer.geo
        self.buf, self.pools, self.geo = buffer, pools, g
        self.H = g.H
        self.Hp = pools.shape("gate")[1]
        assert pools.shape("gate") == (g.H, self.Hp) and pools.shape("up") == (g.H, self.Hp)
        assert pools.shape("down") == (self.Hp, g.H)
        assert g.token_padding % 128 == 0, "the grouped GEMM needs token_padding to be a multiple of 128"
        assert pools.epn == g.epn
        self.overlap_prefetch = overlap_prefetch
        if overlap_backward is None:        # MOONEP_OVERLAP_BACKWARD=0 serialises the backward pass
            overlap_backward = os.environ.get("MOONEP_OVERLAP_BACKWARD", "1") != "0"
        self.overlap_backward = overlap_backward
        if ready_flags is None:             # MOONEP_READY_FLAGS=0: the GEMMs wait for the whole dispatch
            ready_flags = os.environ.get("MOONEP_READY_FLAGS", "1") != "0"
        self.ready_flags = ready_flags
        dev = buffer.hidden_nvsh_buffer_view.device
        self._side = torch.cuda.Stream(device=dev)
        self._opt = torch.cuda.Stream(device=dev)
        self._total_sms = torch.cuda.get_device_properties(dev).multi_processor_count
        self._comm_sms = min(g.num_sms & ~1, self._total_sms - 2)
        self.on_grad_ready = None       # callable(name) -> None, see backward()
        # callable() -> None, called in backward() on the compute stream where a stretch without communication
        # kernels begins (after dgrad(down): SwiGLU backward and two weight-gradient GEMMs follow) -- the
        # place to start work that disturbs them, such as a host-to-device copy of the next batch
        self.on_comm_quiet = None
        self.grads_pending = None       # (projection, event) of a reduction still running after backward()
        # opt-in: backward() may return while the reduction of ``up`` still runs on the comm stream;
        # the caller then calls wait_grads() before it reads those gradients or uses the Buffer again
        self.defer_last_reduction = False
        bf = dict(dtype=torch.bfloat16, device=dev)
        # activations are allocated once; shapes are static (no per-step allocator traffic)
        self._act = torch.zeros(g.NvS, self.Hp, **bf)
        self._gu = torch.zeros(g.NvS, 2 * self.Hp, **bf)
        self._dA = torch.zeros(g.NvS, self.Hp, **bf)
        self._dgu = torch.zeros(g.NvS, 2 * self.Hp, **bf)
        self._x = torch.zeros(g.NvS, g.H, **bf)
        self._w = torch.zeros(g.NvS, dtype=torch.float32, device=dev)
        self.accumulate_grads = False
        # optimizer in the weight-gradient GEMM's epilogue (see ``backward``): learning rate, or None
        self.epilogue_lr = None
        i32 = dict(dtype=torch.int32, device=dev)
        self._upd_mask = torch.zeros(2 * g.epn, **i32)
        self._upd_hit = torch.zeros(g.epn + 1, **i32)
        self._upd_ones = torch.ones(g.R * g.epn, **i32)

    def _update_mask(self, plan):
        return update_mask(plan.experts_to_copy, self.buf.rank, self.geo.epn, self._upd_mask, self._upd_hit, self._upd_ones)

    # weights / grads as [2*epn, in, out]
    def _W(self, n):
        return self.pools.compute_weight(n)

    def _dW(self, n):
        return self.pools.compute_grad(n)

    def forward(self, hidden_sh, route_weights_sk, topk_sk, tokens_per_expert, need_backward: bool = True):
        buf, g, epn = self.buf, self.geo, self.geo.epn
        self._join_deferred()
        if gg.failed(self._act.device):     # a GEMM of an earlier step gave up a wait (host-visible flag, no sync)
            gg.check_status(self._act.device)
        if self.ready_flags:
            return self._forward_flagged(hidden_sh, route_weights_sk, topk_sk, tokens_per_expert, need_backward)
        h_view, w_view, cu, plan = buf.dispatch(hidden_sh, route_weights_sk, topk_sk, tokens_per_expert,
                                                zero_copy=True, router_weights_zero_copy=True)
        ev = None
        if g.R > 1:
            ev = buf.prefetch_weight(plan=plan, async_finish=self.overlap_prefetch, **self.pools.prefetch_kwargs())
        x, w = h_view, w_view
        stashed = None
        if need_backward:       # the shard is overwritten by the down GEMM: keep private copies for wgrad
            main = torch.cuda.current_stream()
            self._side.wait_stream(main)
            with torch.cuda.stream(self._side):
                self._x.copy_(h_view)
                self._w.copy_(w_view)
                stashed = self._side.record_event()
        gu = self._gu if need_backward else None
        Wg, Wu, Wd = self._W("gate"), self._W("up"), self._W("down")
        if ev is not None:
            gg.gate_up(x, Wg, Wu, cu, self._act, gu, row_scale=w, groups=(0, epn))
            torch.cuda.current_stream().wait_event(ev)
            gg.gate_up(x, Wg, Wu, cu, self._act, gu, row_scale=w, groups=(epn, 2 * epn))
        else:
            gg.gate_up(x, Wg, Wu, cu, self._act, gu, row_scale=w)
        return self._forward_tail(plan, cu, stashed, need_backward)

    def _forward_flagged(self, hidden_sh, route_weights_sk, topk_sk, tokens_per_expert, need_backward):
        """Forward pass with tile-ready flags: see the module docstring."""
        buf, g, epn = self.buf, self.geo, self.geo.epn
        main, comm = torch.cuda.current_stream(), buf.comm_stream
        x, w, cu, plan, ready, ev_disp = buf.dispatch_ready(hidden_sh, route_weights_sk, topk_sk, tokens_per_expert)
        if g.R > 1:     # queued on the comm stream behind the dispatch kernel
            buf.prefetch_weight(plan=plan, async_finish=True, **self.pools.prefetch_kwargs())
        stashed = None
        if need_backward:       # private copies for wgrad, taken as soon as the dispatch kernel has finished
            self._side.wait_event(ev_disp)
            with torch.cuda.stream(self._side):
                self._x.copy_(x)
                self._w.copy_(w)
                stashed = self._side.record_event()
        gu = self._gu if need_backward else None
        Wg, Wu = self._W("gate"), self._W("up")
        # one GEMM over all groups, two launches on one ticket counter -- now, on the SMs the dispatch
        # kernel leaves free, and behind dispatch (+ prefetch) on the comm stream for the rest. Token
        # tiles are taken as their ready flags come up; the groups of prefetched experts (the last ones
        # in tile order) additionally wait for their slot's flag, not for the whole prefetch.
        slots = buf.slot_ready() if g.R > 1 else None
        tk = gg.Ticket(self._act.device, self._total_sms)
        free = min(ready.free_sms, self._total_sms - self._comm_sms)
        gg.gate_up(x, Wg, Wu, cu, self._act, gu, row_scale=w, num_ctas=free, ticket=tk, ready=ready, slots=slots)
        with torch.cuda.stream(comm):
            gg.gate_up(x, Wg, Wu, cu, self._act, gu, row_scale=w, num_ctas=self._total_sms - free, ticket=tk,
                       ready=ready, slots=slots)
            joined = comm.record_event()
        main.wait_event(joined)
        return self._forward_tail(plan, cu, stashed, need_backward)

    def _forward_tail(self, plan, cu, stashed, need_backward):
        buf, g = self.buf, self.geo
        Wd = self._W("down")
        if stashed is not None:
            torch.cuda.current_stream().wait_event(stashed)
        if g.off_push:
            # push-combine: the down GEMM's epilogue sends every row to its source rank while the
            # GEMM is still running; what is left of the combine is a barrier and a local sum
            gg.down(self._act, Wd, cu, buf.hidden_nvsh_buffer_view, push=buf.push_target())
            out, _, _ = buf.combine_pushed()
        else:
            gg.down(self._act, Wd, cu, buf.hidden_nvsh_buffer_view)
            out, _, _ = buf.combine(plan=plan, hidden_nvsh=buf.hidden_nvsh_buffer_view, zero_copy=True)
        ctx = MoEContext(plan, cu, self._x, self._w, self._act, self._gu) if need_backward else None
        return out, ctx

    def _optimizer(self, name: str, *after):
        """Run the integrator's per-projection optimizer hook on the optimizer stream once the
        events / streams in ``after`` are done."""
        if self.on_grad_ready is None:
            return
        for a in after:
            if isinstance(a, torch.cuda.Event):
                self._opt.wait_event(a)
            else:
                self._opt.wait_stream(a)
        with torch.cuda.stream(self._opt):
            self.on_grad_ready(name)

    def _beside_comm(self, launch):
        """Issue one grouped GEMM that shares the GPU with the communication kernel just queued on
        the comm stream: ``launch(num_ctas, ticket)`` is called twice with one ticket counter --
        on the current stream for the SMs the communication kernel leaves free, and on the comm
        stream behind that kernel for the SMs it gives back -- so the two launches split the
        GEMM's tiles dynamically.  Returns the event that completes the second launch."""
        tk = gg.Ticket(self._act.device, self._total_sms)
        launch(self._total_sms - self._comm_sms, tk)
        comm = self.buf.comm_stream
        with torch.cuda.stream(comm):
            launch(self._comm_sms, tk)
            return comm.record_event()

    def backward(self, ctx: MoEContext, grad_out_sh):
        """Order of work (``overlap_backward``): the weight-grad GEMMs of ``down`` and ``gate`` come
        first, so that their cross-rank reduction runs on the comm stream beside dgrad(gate/up); the
        combine of the input grads then runs beside wgrad(up); only the reduction of ``up`` is
        exposed.  A GEMM that shares the GPU with a communication kernel is split over two launches
        with a common ticket counter (``_beside_comm``).
        ``on_grad_ready(name)``, if set, is called on a side stream as soon as the local gradient of
        projection ``name`` is final and its weights are no longer read (optimizer in backward).
        ``epilogue_lr``, if set: the weight-gradient GEMMs apply ``W -= lr * dW`` in their epilogue for
        every local expert without a replica elsewhere and write no gradient for it (``_upd_mask``);
        each of them runs after the last GEMM that reads its weights (wgrad(gate) moves behind
        dgrad(gate/up), see below).  Replicated experts keep the stored-gradient path -- their gradients
        are reduced across ranks first -- and ``on_grad_ready`` is expected to update exactly those."""
        buf, g, epn, Hp = self.buf, self.geo, self.geo.epn, self.Hp
        acc, ov, multi = self.accumulate_grads, self.overlap_backward, self.geo.R > 1
        self._join_deferred()
        main = torch.cuda.current_stream()
        pools = self.pools
        pair = lambda n: (pools.local_grad(n), pools.reduce_view(n))      # noqa: E731
        Wg, Wu, Wd = self._W("gate"), self._W("up"), self._W("down")
        shard = buf.hidden_nvsh_buffer_view
        # slots shared with other layers hold someone else's experts by now: fetch this layer's again
        # (on the comm stream, behind the dispatch); the dgrad GEMMs wait per slot
        refetch = multi and getattr(pools, "shared", None) is not None
        slots, ev_pf = None, None
        if self.ready_flags and ctx.plan.send_list is not None:
            # dgrad(down) starts on the tiles of the re-dispatched output grad as they complete
            dy, _, _, _, ready, _ = buf.dispatch_ready(grad_out_sh, plan=ctx.plan)
            if refetch:
                ev_pf = buf.prefetch_weight(plan=ctx.plan, async_finish=True, **pools.prefetch_kwargs())
                slots = buf.slot_ready()
            tk = gg.Ticket(self._act.device, self._total_sms)
            free = min(ready.free_sms, self._total_sms - self._comm_sms)
            gg.dgrad(dy, Wd, ctx.cu, self._dA, num_ctas=free, ticket=tk, ready=ready, slots=slots)
            with torch.cuda.stream(buf.comm_stream):
                gg.dgrad(dy, Wd, ctx.cu, self._dA, num_ctas=self._total_sms - free, ticket=tk, ready=ready, slots=slots)
                joined = buf.comm_stream.record_event()
            main.wait_event(joined)
        else:
            dy, _, _, _ = buf.dispatch(grad_out_sh, plan=ctx.plan, zero_copy=True)
            if refetch:
                ev_pf = buf.prefetch_weight(plan=ctx.plan, async_finish=True, **pools.prefetch_kwargs())
                slots = buf.slot_ready()
            gg.dgrad(dy, Wd, ctx.cu, self._dA, slots=slots)
        if ev_pf is not None:
            main.wait_event(ev_pf)      # dgrad(gate/up) further down reads the other two projections' slots
        dw_view = buf.router_weight_buffer_view
        if self.on_comm_quiet is not None:
            self.on_comm_quiet()
        gg.swiglu_bwd(self._dA, ctx.gu, ctx.w_nvs, self._dgu, dw_view, ctx.cu)
        upd = lambda n: None      # noqa: E731
        if self.epilogue_lr is not None:
            assert not acc, "the optimizer cannot sit in the GEMM epilogue while gradients are accumulated"
            mask, lr_e = self._update_mask(ctx.plan), self.epilogue_lr
            upd = lambda n: (self._W(n), lr_e, mask)      # noqa: E731
        gg.wgrad(ctx.act, dy, ctx.cu, self._dW("down"), accumulate=acc, zero_empty_below=epn, update=upd("down"))
        if not multi:
            self._optimizer("down", main)
        dW_gate, dG = self._dW("gate"), self._dgu[:, :Hp]
        # With the optimizer in the epilogues, wgrad(gate) must come after dgrad(gate/up), which reads the gate
        # weights: the order becomes  reduce(down) | dgrad(gate/up),  combine | wgrad(gate),  reduce(gate) |
        # wgrad(up),  reduce(up)  -- every communication kernel still has a GEMM to run beside, except the last.
        gate_late = self.epilogue_lr is not None
        if not gate_late:
            gg.wgrad(ctx.x, dG, ctx.cu, dW_gate, accumulate=acc, zero_empty_below=epn)
        ev_red = None
        if multi:
            # the weight-gradient GEMMs overwrite the slots they use, so consumed slots need no zeroing
            # unless gradients are accumulated over several backward passes
            first = [pair("down")] if gate_late else [pair("down"), pair("gate")]
            ev_red = buf.reduce_grad_subset(ctx.plan, first, async_finish=ov, clear_slots=acc)
            self._optimizer("down", ev_red if ov else main)
        if ov and multi:
            ev = self._beside_comm(lambda n, tk: gg.dgrad_gate_up(self._dgu, Wg, Wu, ctx.cu, shard, num_ctas=n, ticket=tk))
            main.wait_event(ev)
        else:
            gg.dgrad_gate_up(self._dgu, Wg, Wu, ctx.cu, shard)
        if not gate_late:
            self._optimizer("gate", main, *([ev_red] if ev_red is not None else []))
        grad_hidden, grad_w, ev_comb = buf.combine(plan=ctx.plan, hidden_nvsh=shard, route_weights_nvs=dw_view,
                                                   async_finish=ov, zero_copy=True, router_weights_zero_copy=True)
        if gate_late:
            if ov:
                ev = self._beside_comm(lambda n, tk: gg.wgrad(ctx.x, dG, ctx.cu, dW_gate, accumulate=acc, zero_empty_below=epn,
                                                              num_ctas=n, ticket=tk, update=upd("gate")))
                main.wait_event(ev)   # also covers the combine, which precedes that launch on the comm stream
            else:
                gg.wgrad(ctx.x, dG, ctx.cu, dW_gate, accumulate=acc, zero_empty_below=epn, update=upd("gate"))
            ev_red_g = None
            if multi:
                ev_red_g = buf.reduce_grad_subset(ctx.plan, [pair("gate")], async_finish=ov, clear_slots=acc)
        dW_up, dU = self._dW("up"), self._dgu[:, Hp:]
        if ov and (multi or not gate_late):      # a communication kernel was just queued on the comm stream
            ev = self._beside_comm(lambda n, tk: gg.wgrad(ctx.x, dU, ctx.cu, dW_up, accumulate=acc, zero_empty_below=epn,
                                                          num_ctas=n, ticket=tk, update=upd("up")))
            main.wait_event(ev)       # also covers the combine, which precedes that launch on the comm stream
        else:
            gg.wgrad(ctx.x, dU, ctx.cu, dW_up, accumulate=acc, zero_empty_below=epn, update=upd("up"))
        if gate_late:
            self._optimizer("gate", main, *([ev_red_g] if ev_red_g is not None else []))
        self.grads_pending = None
        if multi:
            # the last reduction has nothing of the backward pass left to hide behind: with
            # ``defer_last_reduction`` it is left running on the comm stream and ``wait_grads()`` (or
            # ``wait_grads("up")``) joins it, so an optimizer can update ``down`` and ``gate`` meanwhile
            ev_up = buf.reduce_grad_subset(ctx.plan, [pair("up")], clear_slots=acc,
                                           async_finish=ov and self.defer_last_reduction)
            if ev_up is not None and self.on_grad_ready is None:
                self.grads_pending = ("up", ev_up)
                _DEFERRED.append(self)
        if self.on_grad_ready is not None:
            if multi and ev_up is not None:
                # the deferred reduction is followed by the optimizer hook of ``up`` on the optimizer stream;
                # ``wait_grads`` then joins that stream (and with it the hooks of ``down`` and ``gate``)
                self._opt.wait_event(ev_up)
                with torch.cuda.stream(self._opt):
                    self.on_grad_ready("up")
                    self.grads_pending = ("up", self._opt.record_event())
                _DEFERRED.append(self)
            else:
                self.on_grad_ready("up")
                main.wait_stream(self._opt)
        return grad_hidden, grad_w

    def wait_grads(self, name: str | None = None) -> None:
        """Make the current stream wait until the expert weight gradients written by the last
        ``backward`` are final: all of them (``name=None``) or those of one projection.  Only the
        reduction of ``up`` can still be in flight after ``backward`` returns."""
        if self.grads_pending is not None and name in (None, self.grads_pending[0]):
            torch.cuda.current_stream().wait_event(self.grads_pending[1])
            self.grads_pending = None
            if self in _DEFERRED:
                _DEFERRED.remove(self)

    @staticmethod
    def forget_deferred() -> None:
        """Drop the record of reductions left running (their events belong to a CUDA-graph capture
        that was abandoned, so they can never be waited on); call after a failed capture."""
        for layer in list(_DEFERRED):
            layer.grads_pending = None
        _DEFERRED.clear()

    @staticmethod
    def _join_deferred() -> None:
        """Before any layer queues new communication kernels, the current stream joins every
        reduction that some layer left running.  Communication kernels wait for their peers while
        they hold their SMs, so two of them from different Buffers must never be left to start in
        different orders on different ranks; joining here keeps one global order."""
        for layer in list(_DEFERRED):
            layer.wait_grads()


class _MoEFn(torch.autograd.Function):
    @staticmethod
    def forward(fctx, hidden, route_weights, topk, tpe, layer: ExpertParallelMoE):
        out, ctx = layer.forward(hidden, route_weights, topk, tpe, need_backward=True)
        fctx.layer, fctx.moe_ctx = layer, ctx
        return out

    @staticmethod
    def backward(fctx, grad_out):
        gh, gw = fctx.layer.backward(fctx.moe_ctx, grad_out.contiguous())
        return gh, gw, None, None, None


def moe_apply(layer: ExpertParallelMoE, hidden, route_weights, topk, tpe):
    """Autograd entry: differentiable w.r.t. ``hidden`` and ``route_weights``; expert weight grads
    are written into the pools' fp32 grad views by the backward pass."""
    return _MoEFn.apply(hidden, route_weights, topk, tpe, layer)
