"""Expert-parallel MoE FFN built on ``Buffer`` + the tcgen05 grouped GEMM.

Forward  : dispatch -> [prefetch_weight on the comm stream] -> gate/up GEMM with fused
           SwiGLU and route-weight scaling (local experts first, prefetched experts once their
           weights have landed) -> down GEMM writing straight into the communication shard ->
           combine (zero copy).
Backward : re-dispatch of the output grad with the saved plan -> dgrad(down) + wgrad(down) ->
           SwiGLU backward (also yields the route-weight grads) -> dgrad(gate/up) into the shard
           -> wgrad(gate), wgrad(up) -> combine with the route-weight-grad channel ->
           reduce_grad of the replicated experts.
This is the integration the reference leaves to the training framework (README.md:110-156 of
the reference gives the same operator mapping).  Weights are ``[2*epn, in, out]`` compute views
of an ``ExpertPools``; weight grads are fp32 ``[2*epn, in, out]`` whose tail is the reduce slots.
"""

from __future__ import annotations

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


class ExpertParallelMoE:
    def __init__(self, buffer: Buffer, pools: ExpertPools, overlap_prefetch: bool = True):
        g = buffer.geo
        self.buf, self.pools, self.geo = buffer, pools, g
        self.H = g.H
        self.Hp = pools.shape("gate")[1]
        assert pools.shape("gate") == (g.H, self.Hp) and pools.shape("up") == (g.H, self.Hp)
        assert pools.shape("down") == (self.Hp, g.H)
        assert g.token_padding % 128 == 0, "the grouped GEMM needs token_padding to be a multiple of 128"
        assert pools.epn == g.epn
        self.overlap_prefetch = overlap_prefetch
        dev = buffer.hidden_nvsh_buffer_view.device
        bf = dict(dtype=torch.bfloat16, device=dev)
        # activations are allocated once; shapes are static (no per-step allocator traffic)
        self._act = torch.zeros(g.NvS, self.Hp, **bf)
        self._gu = torch.zeros(g.NvS, 2 * self.Hp, **bf)
        self._dA = torch.zeros(g.NvS, self.Hp, **bf)
        self._dgu = torch.zeros(g.NvS, 2 * self.Hp, **bf)
        self._x = torch.zeros(g.NvS, g.H, **bf)
        self._w = torch.zeros(g.NvS, dtype=torch.float32, device=dev)
        self.accumulate_grads = False

    # weights / grads as [2*epn, in, out]
    def _W(self, n):
        return self.pools.compute_weight(n)

    def _dW(self, n):
        return self.pools.compute_grad(n)

    def forward(self, hidden_sh, route_weights_sk, topk_sk, tokens_per_expert, need_backward: bool = True):
        buf, g, epn = self.buf, self.geo, self.geo.epn
        h_view, w_view, cu, plan = buf.dispatch(hidden_sh, route_weights_sk, topk_sk, tokens_per_expert,
                                                zero_copy=True, router_weights_zero_copy=True)
        ev = None
        if g.R > 1:
            ev = buf.prefetch_weight(plan=plan, async_finish=self.overlap_prefetch, **self.pools.prefetch_kwargs())
        if need_backward:       # the shard is overwritten below: keep private copies for wgrad
            self._x.copy_(h_view)
            self._w.copy_(w_view)
            x, w = self._x, self._w
        else:
            x, w = h_view, w_view
        gu = self._gu if need_backward else None
        Wg, Wu, Wd = self._W("gate"), self._W("up"), self._W("down")
        if ev is not None:
            gg.gate_up(x, Wg, Wu, cu, self._act, gu, row_scale=w, groups=(0, epn))
            torch.cuda.current_stream().wait_event(ev)
            gg.gate_up(x, Wg, Wu, cu, self._act, gu, row_scale=w, groups=(epn, 2 * epn))
        else:
            gg.gate_up(x, Wg, Wu, cu, self._act, gu, row_scale=w)
        gg.down(self._act, Wd, cu, buf.hidden_nvsh_buffer_view)
        out, _, _ = buf.combine(plan=plan, hidden_nvsh=buf.hidden_nvsh_buffer_view, zero_copy=True)
        ctx = MoEContext(plan, cu, x, w, self._act, self._gu) if need_backward else None
        return out, ctx

    def backward(self, ctx: MoEContext, grad_out_sh):
        buf, g, epn, Hp = self.buf, self.geo, self.geo.epn, self.Hp
        acc = self.accumulate_grads
        dy, _, _, _ = buf.dispatch(grad_out_sh, plan=ctx.plan, zero_copy=True)
        Wg, Wu, Wd = self._W("gate"), self._W("up"), self._W("down")
        gg.dgrad(dy, Wd, ctx.cu, self._dA)
        gg.wgrad(ctx.act, dy, ctx.cu, self._dW("down"), accumulate=acc, zero_empty_below=epn)
        dw_view = buf.router_weight_buffer_view
        gg.swiglu_bwd(self._dA, ctx.gu, ctx.w_nvs, self._dgu, dw_view, ctx.cu)
        gg.dgrad_gate_up(self._dgu, Wg, Wu, ctx.cu, buf.hidden_nvsh_buffer_view)
        gg.wgrad(ctx.x, self._dgu[:, :Hp], ctx.cu, self._dW("gate"), accumulate=acc, zero_empty_below=epn)
        gg.wgrad(ctx.x, self._dgu[:, Hp:], ctx.cu, self._dW("up"), accumulate=acc, zero_empty_below=epn)
        grad_hidden, grad_w, _ = buf.combine(plan=ctx.plan, hidden_nvsh=buf.hidden_nvsh_buffer_view,
                                             route_weights_nvs=dw_view, zero_copy=True, router_weights_zero_copy=True)
        if g.R > 1:
            buf.reduce_grad(plan=ctx.plan, **self.pools.reduce_kwargs())
        return grad_hidden, grad_w


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
