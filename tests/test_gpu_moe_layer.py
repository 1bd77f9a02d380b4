"""The expert-parallel MoE layer (dispatch -> grouped GEMM -> combine, forward and backward)
against a dense fp32 PyTorch implementation of the same top-k MoE."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_moe_layer_matches_dense_reference(cuda_device):
    from moonep_b200.models.moe_block import MoEBlock, MoEConfig
    cfg = MoEConfig("t", H=256, Hp=256, K=2, epn=4, shared_experts=0, S=192)
    blk = MoEBlock(cfg, num_sms=4, seed=3)
    torch.manual_seed(1)
    x = (torch.randn(cfg.S, cfg.H, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
    w, topk, tpe = blk.route(x.detach())
    wl = w.detach().clone().requires_grad_(True)
    from moonep_b200.moe_layer import moe_apply
    y = moe_apply(blk.moe, x, wl, topk, tpe)
    gy = (torch.randn_like(y.float()) * 0.1).to(torch.bfloat16)
    y.backward(gy)
    torch.cuda.synchronize()
    blk.buf.check()

    # dense fp32 reference
    xf = x.detach().float().requires_grad_(True)
    wf = w.detach().clone().requires_grad_(True)
    Wg = blk.pools.local_weight("gate").float().requires_grad_(True)
    Wu = blk.pools.local_weight("up").float().requires_grad_(True)
    Wd = blk.pools.local_weight("down").float().requires_grad_(True)
    ref = torch.zeros(cfg.S, cfg.H, device="cuda")
    for k in range(cfg.K):
        e = topk[:, k].long()
        h = torch.nn.functional.silu(torch.einsum("sh,shp->sp", xf, Wg[e])) * torch.einsum("sh,shp->sp", xf, Wu[e])
        ref = ref + wf[:, k:k + 1] * torch.einsum("sp,sph->sh", h, Wd[e])
    ref.backward(gy.float())

    def rel(a, b):
        return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))

    assert rel(y, ref) < 2e-2, f"forward {rel(y, ref)}"
    assert rel(x.grad, xf.grad) < 3e-2, f"grad hidden {rel(x.grad, xf.grad)}"
    assert rel(wl.grad, wf.grad) < 3e-2, f"grad route weights {rel(wl.grad, wf.grad)}"
    for n, W in (("gate", Wg), ("up", Wu), ("down", Wd)):
        assert rel(blk.pools.local_grad(n), W.grad) < 3e-2, f"grad {n} {rel(blk.pools.local_grad(n), W.grad)}"
    blk.destroy()


def test_smoke_step(cuda_device):
    from moonep_b200.models.moe_block import smoke_step
    loss = smoke_step()
    assert loss == loss
