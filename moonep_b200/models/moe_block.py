"""MoE transformer FFN blocks of the model families the benchmarks name.

``MoEBlock`` = router (softmax top-k over a dense gate projection) + expert-parallel routed
experts (SwiGLU) + optional dense shared expert, with a fused SGD step for benchmarks.  Shapes:

    deepseek_v3   H=7168, H'=2048, K=8, epn=32 (E=256 at EP=8)
    kimi_k2       H=7168, H'=2048, K=8, epn=48 (E=384 at EP=8), one shared expert
    qwen3_30b_a3b H=2048, H'=768,  K=8, epn=16 (E=128 at EP=8)

The reference library contains no model code; these blocks exist so that its headline
benchmark ("MoE-layer step vs maxvio") can be run end to end through this package.
"""

from __future__ import annotations

import os
from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..api import Buffer
from ..moe_layer import ExpertParallelMoE, moe_apply
from ..ops import grouped_gemm as gg
from ..pools import ExpertPools


@dataclass(frozen=True)
class MoEConfig:
    name: str
    H: int
    Hp: int
    K: int
    epn: int
    shared_experts: int = 0
    S: int = 4096
    token_padding: int = 128


CONFIGS = {
    "deepseek_v3": MoEConfig("deepseek_v3", 7168, 2048, 8, 32),
    "kimi_k2": MoEConfig("kimi_k2", 7168, 2048, 8, 48, shared_experts=1),
    "qwen3_30b_a3b": MoEConfig("qwen3_30b_a3b", 2048, 768, 8, 16, S=8192),
    "tiny": MoEConfig("tiny", 256, 256, 2, 2, shared_experts=1, S=128),
}


class MoEBlock:
    """One MoE FFN block on this rank of the EP group (weights random-init N(0, 0.02))."""

    def __init__(self, cfg: MoEConfig, world: int = 1, rank: int = 0, group=None, num_sms: int = 32, seed: int = 0,
                 router_skew: float = 0.0, buffer: Buffer | None = None, shared_slots=None):
        """``buffer`` / ``shared_slots``: a ``Buffer`` and a ``pools.SharedSlots`` that several blocks of
        one model use in turn (the communication buffers and the prefetch / reduce slots are scratch
        between a layer's dispatch and its combine, so a model needs them once); without them the
        block creates its own."""
        self.cfg, self.world, self.rank = cfg, world, rank
        dev = torch.device("cuda", torch.cuda.current_device())
        self.E = cfg.epn * world
        # the down GEMM's epilogue sends its rows to their source ranks itself; costs a [S*K, H]
        # receive area per rank (MOONEP_PUSH_COMBINE=0: plain stores, then the combine pulls)
        push = os.environ.get("MOONEP_PUSH_COMBINE", "1") != "0"
        self._own_buffer = buffer is None
        self.buf = buffer if buffer is not None else Buffer(cfg.S, cfg.H, cfg.K, self.E, world, num_sms=num_sms,
                                                            token_padding=cfg.token_padding, group=group, push_combine=push)
        self.pools = ExpertPools(cfg.epn, (cfg.H, cfg.Hp), (cfg.H, cfg.Hp), (cfg.Hp, cfg.H), group=group, with_grads=True,
                                 shared=shared_slots if world > 1 else None)
        g = torch.Generator(device=dev).manual_seed(seed * 7919 + rank)
        for n in ("gate", "up", "down"):
            w = self.pools.local_weight(n)
            w.copy_((torch.randn(w.shape, device=dev, generator=g) * 0.02).to(torch.bfloat16))
            self.pools.compute_grad(n).zero_()
        gs = torch.Generator(device=dev).manual_seed(seed)       # router is replicated: same on all ranks
        self.router = (torch.randn(cfg.H, self.E, device=dev, generator=gs) * 0.02).to(torch.bfloat16).requires_grad_(True)
        # a per-expert bias added to the logits skews the routing (maxvio sweeps)
        self.router_bias = (torch.randn(self.E, device=dev, generator=gs) * router_skew).float()
        self.shared = None
        if cfg.shared_experts:
            hs = cfg.Hp * cfg.shared_experts
            self.shared = [(torch.randn(cfg.H, 2 * hs, device=dev, generator=g) * 0.02).to(torch.bfloat16).requires_grad_(True),
                           (torch.randn(hs, cfg.H, device=dev, generator=g) * 0.02).to(torch.bfloat16).requires_grad_(True)]
        self.moe = ExpertParallelMoE(self.buf, self.pools)
        # sgd_step() joins the last gradient reduction before it updates ``up``
        self.moe.defer_last_reduction = os.environ.get("MOONEP_DEFER_LAST_REDUCTION", "1") != "0"
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier(group=group)

    def route(self, hidden):
        cfg = self.cfg
        logits = (hidden @ self.router).float() + self.router_bias
        probs = torch.softmax(logits, dim=-1)
        w, topk = torch.topk(probs, cfg.K, dim=-1)
        w = (w / w.sum(dim=-1, keepdim=True)).contiguous()
        topk = topk.to(torch.int32).contiguous()
        tpe = torch.zeros(self.E, dtype=torch.int32, device=hidden.device)
        tpe.scatter_add_(0, topk.reshape(-1).long(), torch.ones(topk.numel(), dtype=torch.int32, device=hidden.device))
        return w, topk, tpe

    def forward(self, hidden):
        w, topk, tpe = self.route(hidden)
        out = moe_apply(self.moe, hidden, w, topk, tpe)
        if self.shared is not None:
            gu = hidden @ self.shared[0]
            hs = gu.shape[1] // 2
            out = out + (torch.nn.functional.silu(gu[:, :hs]) * gu[:, hs:]) @ self.shared[1]
        return out

    def parameters(self):
        ps = [self.router]
        if self.shared is not None:
            ps += self.shared
        return ps

    def fuse_optimizer(self, lr: float | None, in_epilogue: bool = False):
        """Apply the experts' SGD update inside the backward pass: each projection is updated on a
        side stream as soon as its gradient is final (``ExpertParallelMoE.on_grad_ready``), beside
        the GEMMs that are still running.  ``None`` switches back to updating in ``sgd_step``.

        ``in_epilogue``: the experts are updated by their weight-gradient GEMMs themselves
        (``wgrad(update=...)``: no fp32 gradient is written or read back for an expert whose gradient is
        complete on this rank); the side-stream kernel then only covers the experts that have replicas on
        other ranks, whose gradients are reduced first.  Same arithmetic, same result."""
        self._fused_lr = lr
        moe = self.moe
        # shapes the CTA-pair weight-gradient kernel does not cover fall back to the stand-alone kernels
        in_epilogue = in_epilogue and all(gg.wgrad_update_supported(*self.pools.shape(n)) for n in ("gate", "up", "down"))
        moe.epilogue_lr = lr if (in_epilogue and lr is not None) else None
        if lr is None:
            moe.on_grad_ready = None
        elif moe.epilogue_lr is None:
            moe.on_grad_ready = lambda n: gg.sgd_step(self.pools.local_weight(n), self.pools.local_grad(n), lr)
        else:
            moe.on_grad_ready = lambda n: gg.sgd_step_groups(self.pools.local_weight(n), self.pools.local_grad(n), lr,
                                                             moe._upd_mask, want=False)

    def sgd_step(self, lr: float):
        if self.moe.on_grad_ready is None:
            for n in ("down", "gate", "up"):     # ``up`` last: its cross-rank reduction may still be running
                self.moe.wait_grads(n)
                gg.sgd_step(self.pools.local_weight(n), self.pools.local_grad(n), lr)
        else:
            assert lr == self._fused_lr, "the experts were already updated with another learning rate"
            self.moe.wait_grads()       # the last reduction and the update behind it may still be running
        with torch.no_grad():
            for p in self.parameters():
                if p.grad is not None:
                    p.add_(p.grad.to(p.dtype), alpha=-lr)
                    p.grad = None

    def destroy(self):
        self.moe.wait_grads()        # nothing of this layer may still be queued on the comm stream
        self.pools.destroy()
        if self._own_buffer:
            self.buf.destroy()


def smoke_step() -> float:
    """One tiny forward + backward + SGD step on the current device (single rank)."""
    torch.manual_seed(0)
    blk = MoEBlock(CONFIGS["tiny"], num_sms=4)
    x = torch.randn(blk.cfg.S, blk.cfg.H, device="cuda").to(torch.bfloat16).requires_grad_(True)
    y = blk.forward(x)
    loss = (y.float() ** 2).mean()
    loss.backward()
    blk.sgd_step(1e-3)
    torch.cuda.synchronize()
    blk.buf.check()
    gg.check_status()
    assert x.grad is not None and torch.isfinite(x.grad.float()).all() and torch.isfinite(loss)
    v = float(loss)
    blk.destroy()
    return v
