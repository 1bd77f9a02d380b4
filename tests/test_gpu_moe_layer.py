"""The expert-parallel MoE layer (dispatch -> grouped GEMM -> combine, forward and backward)
against a dense fp32 PyTorch implementation of the same top-k MoE."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("ready_flags", [False, True], ids=["barrier", "flags"])
@pytest.mark.parametrize("push_combine", [False, True], ids=["pull", "push"])
def test_moe_layer_matches_dense_reference(push_combine, ready_flags, cuda_device, monkeypatch):
    from moonep_b200.models.moe_block import MoEBlock, MoEConfig
    monkeypatch.setenv("MOONEP_PUSH_COMBINE", "1" if push_combine else "0")
    monkeypatch.setenv("MOONEP_READY_FLAGS", "1" if ready_flags else "0")
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


def _train(blk, xs, lr, steps, graphed):
    """``steps`` SGD steps on the inputs ``xs`` (used in turn); returns the losses."""
    from moonep_b200.utils import GraphedSteps

    def step(x):
        x.requires_grad_(True)
        loss = (blk.forward(x).float() ** 2).sum()        # a sum: the updates must be visible in bf16 weights
        loss.backward()
        blk.sgd_step(lr)
        x.grad = None
        return loss.detach()

    losses = []
    if graphed:
        gs = GraphedSteps(step, xs)
        for i in range(steps):
            gs.replay(i)
            torch.cuda.synchronize()
            losses.append(float(gs.host_losses[i % len(xs)][0]))
    else:
        for i in range(steps):
            losses.append(float(step(xs[i % len(xs)])))
    torch.cuda.synchronize()
    blk.buf.check()
    return losses


@pytest.mark.parametrize("optimizer_in_backward", [False, True])
def test_captured_steps_match_eager_steps(optimizer_in_backward, cuda_device):
    """A step captured as a CUDA graph and replayed gives the losses and weights of the same steps
    launched from Python (planner epochs, barrier state and tile counters all live on the device),
    with the optimizer after or inside the backward pass."""
    from moonep_b200.models.moe_block import MoEBlock, MoEConfig
    from moonep_b200.ops import grouped_gemm as gg
    cfg = MoEConfig("t", H=256, Hp=256, K=2, epn=4, shared_experts=1, S=192)
    g = torch.Generator(device="cuda").manual_seed(5)
    xs = [(torch.randn(cfg.S, cfg.H, device="cuda", generator=g) * 0.5).to(torch.bfloat16) for _ in range(2)]
    out = []
    for graphed in (False, True):
        blk = MoEBlock(cfg, num_sms=4, seed=3)
        if optimizer_in_backward:
            blk.fuse_optimizer(1e-2)
        _train(blk, [x.clone() for x in xs], 1e-2, 2, graphed=False)          # warm-up, eager in both runs
        losses = _train(blk, [x.clone() for x in xs], 1e-2, 5, graphed=graphed)
        gg.check_status()
        out.append((losses, [blk.pools.local_weight(n).clone() for n in ("gate", "up", "down")]))
        blk.destroy()
    (l0, w0), (l1, w1) = out
    assert all(abs(a - b) <= 1e-3 * abs(a) + 1e-6 for a, b in zip(l0, l1)), (l0, l1)
    assert l0[0] != l0[2], "the weights must actually be trained (same input, two steps later)"
    for a, b in zip(w0, w1):
        assert torch.equal(a, b)


def test_captured_steps_stage_the_next_batch(cuda_device):
    """``GraphedSteps(host_inputs=...)``: every replay copies the next step's batch from pinned host memory
    inside its own graph, starting where the step says (here: before the optimizer).  Batches that the host
    rewrites between replays must arrive, and losses and weights must equal those of eager steps on the
    same sequence of batches."""
    from moonep_b200.models.moe_block import MoEBlock, MoEConfig
    from moonep_b200.ops import grouped_gemm as gg
    from moonep_b200.utils import GraphedSteps
    cfg = MoEConfig("t", H=256, Hp=256, K=2, epn=4, shared_experts=1, S=192)
    g = torch.Generator().manual_seed(6)
    batches = [(torch.randn(cfg.S, cfg.H, generator=g) * 0.5).to(torch.bfloat16) for _ in range(6)]
    lr = 1e-2

    def make_step(blk):
        def step(x, stage_next=None):
            x.requires_grad_(True)
            loss = (blk.forward(x).float() ** 2).sum()
            loss.backward()
            if stage_next is not None:
                stage_next()
            blk.sgd_step(lr)
            x.grad = None
            return loss.detach()
        return step

    out = []
    for graphed in (False, True):
        blk = MoEBlock(cfg, num_sms=4, seed=3)
        step = make_step(blk)
        for i in range(2):
            step(batches[i].cuda())                                         # warm-up, eager in both runs
        losses = []
        if graphed:
            host = [batches[0].clone().pin_memory(), batches[1].clone().pin_memory()]
            dev = [torch.empty_like(batches[0], device="cuda") for _ in range(2)]
            gs = GraphedSteps(step, dev, host_inputs=host)                  # capture runs no kernel
            dev[0].detach().copy_(host[0])                                  # the first batch is the caller's
            for i in range(len(batches)):
                if i + 1 < len(batches):
                    host[(i + 1) % 2].copy_(batches[i + 1])                 # the loader refills the pinned buffer
                gs.replay(i)
                torch.cuda.synchronize()
                losses.append(float(gs.host_losses[i % 2][0]))
                if i + 1 < len(batches):
                    assert torch.equal(dev[(i + 1) % 2].detach().cpu(), batches[i + 1]), f"batch {i + 1} did not arrive"
        else:
            for b in batches:
                losses.append(float(step(b.cuda())))
        torch.cuda.synchronize()
        blk.buf.check(); gg.check_status()
        out.append((losses, [blk.pools.local_weight(n).clone() for n in ("gate", "up", "down")]))
        blk.destroy()
    (l0, w0), (l1, w1) = out
    assert all(abs(a - b) <= 1e-3 * abs(a) + 1e-6 for a, b in zip(l0, l1)), (l0, l1)
    for a, b in zip(w0, w1):
        assert torch.equal(a, b)


@pytest.mark.parametrize("overlap", ["1", "0"], ids=["overlapped_backward", "serial_backward"])
@pytest.mark.parametrize("graphed", [False, True], ids=["eager", "captured"])
def test_optimizer_in_the_wgrad_epilogue_matches_the_stand_alone_optimizer(graphed, overlap, cuda_device, monkeypatch):
    """``fuse_optimizer(lr, in_epilogue=True)``: the experts are updated by their weight-gradient GEMMs
    (wgrad(gate) moves behind dgrad(gate/up) for that).  Losses and weights must equal those of
    the same steps with the optimizer after the backward pass, bit for bit."""
    from moonep_b200.models.moe_block import MoEBlock, MoEConfig
    from moonep_b200.ops import grouped_gemm as gg
    monkeypatch.setenv("MOONEP_OVERLAP_BACKWARD", overlap)
    cfg = MoEConfig("t", H=256, Hp=256, K=2, epn=4, shared_experts=1, S=192)
    g = torch.Generator(device="cuda").manual_seed(8)
    xs = [(torch.randn(cfg.S, cfg.H, device="cuda", generator=g) * 0.5).to(torch.bfloat16) for _ in range(2)]
    out = []
    for in_epilogue in (False, True):
        blk = MoEBlock(cfg, num_sms=4, seed=3)
        if in_epilogue:
            blk.fuse_optimizer(1e-2, in_epilogue=True)
        _train(blk, [x.clone() for x in xs], 1e-2, 2, graphed=False)
        losses = _train(blk, [x.clone() for x in xs], 1e-2, 5, graphed=graphed)
        gg.check_status()
        out.append((losses, [blk.pools.local_weight(n).clone() for n in ("gate", "up", "down")]))
        if in_epilogue:
            assert int(blk.moe._upd_mask[:cfg.epn].sum()) == cfg.epn, "one rank: every expert takes the fused path"
        blk.destroy()
    (l0, w0), (l1, w1) = out
    assert l0 == l1, (l0, l1)
    assert l0[0] != l0[2]
    for a, b in zip(w0, w1):
        assert torch.equal(a, b)
