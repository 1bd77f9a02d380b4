"""Numerics of the tcgen05 grouped GEMM against a plain fp32 PyTorch reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(G, rows_per_group, K, N, seed=0, dev="cuda"):
    g = torch.Generator(device=dev).manual_seed(seed)
    cu, tot = [], 0
    for r in rows_per_group:
        tot += r
        cu.append(tot)
    cu = torch.tensor(cu, dtype=torch.int32, device=dev)
    rows = tot + 128          # extra undefined tail rows must not be touched
    x = (torch.randn(rows, K, device=dev, generator=g) * 0.5).to(torch.bfloat16)
    return cu, tot, rows, x, g


def _group_slices(rows_per_group):
    s = 0
    for gi, r in enumerate(rows_per_group):
        yield gi, s, s + r
        s += r


def _relerr(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


@pytest.mark.parametrize("tile_order", ["static", "dynamic"])
@pytest.mark.parametrize("pair_kernels", [False, True], ids=["1cta", "cta_pairs"])
@pytest.mark.parametrize("rpg", [[128, 0, 256, 128], [384, 128, 0, 0, 128, 256]])
def test_gate_up_down(rpg, pair_kernels, tile_order, cuda_device, monkeypatch):
    from moonep_b200.ops import grouped_gemm as gg
    monkeypatch.setenv("MOONEP_GEMM_DYNAMIC", "1" if tile_order == "dynamic" else "0")
    monkeypatch.setenv("MOONEP_GEMM_2CTA", "1" if pair_kernels else "0")
    G, K, N = len(rpg), 256, 256
    cu, tot, rows, x, g = _setup(G, rpg, K, N)
    wg = (torch.randn(G, K, N, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    wu = (torch.randn(G, K, N, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    wd = (torch.randn(G, N, K, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    scale = torch.rand(rows, device="cuda", generator=g) + 0.5
    act = torch.full((rows, N), 7.0, dtype=torch.bfloat16, device="cuda")
    gu = torch.full((rows, 2 * N), 7.0, dtype=torch.bfloat16, device="cuda")
    gg.gate_up(x, wg, wu, cu, act, gu, row_scale=scale)
    y = torch.full((rows, K), 7.0, dtype=torch.bfloat16, device="cuda")
    gg.down(act, wd, cu, y)
    torch.cuda.synchronize()
    gg.check_status()
    for gi, a, b in _group_slices(rpg):
        if a == b:
            continue
        xf = x[a:b].float()
        gr, ur = xf @ wg[gi].float(), xf @ wu[gi].float()
        ar = torch.nn.functional.silu(gr) * ur * scale[a:b, None]
        assert _relerr(gu[a:b, :N], gr) < 1e-2 and _relerr(gu[a:b, N:], ur) < 1e-2, f"group {gi}: pre-activations"
        assert _relerr(act[a:b], ar) < 1.5e-2, f"group {gi}: swiglu"
        yr = act[a:b].float() @ wd[gi].float()
        assert _relerr(y[a:b], yr) < 1e-2, f"group {gi}: down"
    assert (act[tot:] == 7.0).all() and (y[tot:] == 7.0).all(), "rows beyond cu_seqlens[-1] were written"


@pytest.mark.parametrize("tile_order", ["static", "dynamic"])
@pytest.mark.parametrize("pair_kernels", [False, True], ids=["1cta", "cta_pairs"])
def test_dgrad_and_wgrad(pair_kernels, tile_order, cuda_device, monkeypatch):
    from moonep_b200.ops import grouped_gemm as gg
    monkeypatch.setenv("MOONEP_GEMM_DYNAMIC", "1" if tile_order == "dynamic" else "0")
    monkeypatch.setenv("MOONEP_GEMM_2CTA", "1" if pair_kernels else "0")
    monkeypatch.setenv("MOONEP_WGRAD_2CTA", "1" if pair_kernels else "0")
    rpg = [256, 128, 0, 384]
    G, H, Hp = len(rpg), 256, 256
    cu, tot, rows, x, g = _setup(G, rpg, H, Hp, seed=1)
    wg = (torch.randn(G, H, Hp, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    wu = (torch.randn(G, H, Hp, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    wd = (torch.randn(G, Hp, H, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    dy = (torch.randn(rows, H, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    dgu = (torch.randn(rows, 2 * Hp, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    dA = torch.zeros(rows, Hp, dtype=torch.bfloat16, device="cuda")
    gg.dgrad(dy, wd, cu, dA)
    dx = torch.zeros(rows, H, dtype=torch.bfloat16, device="cuda")
    gg.dgrad_gate_up(dgu, wg, wu, cu, dx)
    dWg = torch.full((G, H, Hp), 3.0, device="cuda")
    dWu = torch.full((G, H, Hp), 3.0, device="cuda")
    gg.wgrad(x, dgu[:, :Hp], cu, dWg, accumulate=False)
    gg.wgrad(x, dgu[:, Hp:], cu, dWu, accumulate=True)
    dWz = torch.full((G, H, Hp), 3.0, device="cuda")
    gg.wgrad(x, dgu[:, :Hp], cu, dWz, accumulate=False, zero_empty_below=G)
    torch.cuda.synchronize()
    gg.check_status()
    for gi, a, b in _group_slices(rpg):
        if a == b:
            assert (dWg[gi] == 3.0).all() and (dWu[gi] == 3.0).all(), "empty group's grads must stay untouched"
            assert (dWz[gi] == 0.0).all(), "empty group must be zeroed when requested"
            continue
        assert _relerr(dA[a:b], dy[a:b].float() @ wd[gi].float().T) < 1e-2, f"group {gi}: dgrad"
        ref = dgu[a:b, :Hp].float() @ wg[gi].float().T + dgu[a:b, Hp:].float() @ wu[gi].float().T
        assert _relerr(dx[a:b], ref) < 1e-2, f"group {gi}: dgrad gate/up"
        assert _relerr(dWg[gi], x[a:b].float().T @ dgu[a:b, :Hp].float()) < 2e-3, f"group {gi}: wgrad"
        assert _relerr(dWu[gi], 3.0 + x[a:b].float().T @ dgu[a:b, Hp:].float()) < 2e-3, f"group {gi}: wgrad accumulate"


def test_swiglu_bwd(cuda_device):
    from moonep_b200.ops import grouped_gemm as gg
    rows, Hp = 256, 128
    g = torch.Generator(device="cuda").manual_seed(2)
    cu = torch.tensor([128, 256], dtype=torch.int32, device="cuda")
    gu = torch.randn(rows, 2 * Hp, device="cuda", generator=g).to(torch.bfloat16)
    dA = torch.randn(rows, Hp, device="cuda", generator=g).to(torch.bfloat16)
    w = torch.rand(rows, device="cuda", generator=g)
    dgu = torch.zeros(rows, 2 * Hp, dtype=torch.bfloat16, device="cuda")
    dw = torch.zeros(rows, device="cuda")
    gg.swiglu_bwd(dA, gu, w, dgu, dw, cu)
    torch.cuda.synchronize()
    gf = gu[:, :Hp].float().requires_grad_(True)
    uf = gu[:, Hp:].float().requires_grad_(True)
    wf = w.clone().requires_grad_(True)
    act = wf[:, None] * torch.nn.functional.silu(gf) * uf
    act.backward(dA.float())
    assert _relerr(dgu[:, :Hp], gf.grad) < 1e-2 and _relerr(dgu[:, Hp:], uf.grad) < 1e-2
    assert _relerr(dw, wf.grad) < 1e-3


def test_sgd(cuda_device):
    from moonep_b200.ops import grouped_gemm as gg
    gen = torch.Generator(device="cuda").manual_seed(11)
    p = torch.randn(4096, device="cuda", generator=gen).to(torch.bfloat16)
    g = torch.randn(4096, device="cuda", generator=gen)
    ref = (p.float() - 0.1 * g).to(torch.bfloat16).float()
    gg.sgd_step(p, g, 0.1)
    torch.cuda.synchronize()
    # the kernel contracts p - lr*g into one fused multiply-add, the fp32 reference rounds twice:
    # a result may land on the neighbouring bf16 value when it sits on a rounding boundary
    diff = (p.float() - ref).abs()
    assert (diff <= ref.abs() * 2.0 ** -7).all(), "more than one bf16 ulp away from the fp32 reference"
    assert (diff != 0).float().mean() < 0.01


@pytest.mark.parametrize("tile_order", ["static", "dynamic"])
def test_wgrad_with_the_optimizer_in_its_epilogue(tile_order, cuda_device, monkeypatch):
    """``wgrad(update=(W, lr, mask))``: groups with a non-zero mask word get ``W -= lr * dW`` and no gradient
    (bit for bit what wgrad + sgd_step give), the others get their gradient and keep their weights; the
    masked stand-alone update covers exactly the complement.  fp32 reference for the gradient itself."""
    from moonep_b200.ops import grouped_gemm as gg
    monkeypatch.setenv("MOONEP_GEMM_DYNAMIC", "1" if tile_order == "dynamic" else "0")
    rpg = [256, 128, 0, 384, 128, 0]
    G, H, Hp, lr = len(rpg), 512, 256, 0.05
    cu, tot, rows, x, g = _setup(G, rpg, H, Hp, seed=4)
    dy = (torch.randn(rows, Hp, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    W0 = (torch.randn(G, H, Hp, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    mask = torch.tensor([1, 0, 1, 1, 0, 0], dtype=torch.int32, device="cuda")
    # reference: plain wgrad, then the stand-alone optimizer on the masked groups
    dW_ref = torch.full((G, H, Hp), 7.0, device="cuda")
    gg.wgrad(x, dy, cu, dW_ref, accumulate=False, zero_empty_below=G)
    W_ref = W0.clone()
    gg.sgd_step_groups(W_ref, dW_ref, lr, mask, want=True)
    # fused
    W = W0.clone()
    dW = torch.full((G, H, Hp), 7.0, device="cuda")
    gg.wgrad(x, dy, cu, dW, accumulate=False, zero_empty_below=G, update=(W, lr, mask))
    torch.cuda.synchronize()
    gg.check_status()
    for gi, a, b in _group_slices(rpg):
        if int(mask[gi]):
            assert torch.equal(W[gi], W_ref[gi]), f"group {gi}: fused update differs from wgrad + sgd"
            assert (dW[gi] == 7.0).all(), f"group {gi}: an updated group must not write its gradient"
            if a == b:
                assert torch.equal(W[gi], W0[gi]), "an empty group must keep its weights"
            else:
                assert not torch.equal(W[gi], W0[gi])
                ref = (W0[gi].float() - lr * (x[a:b].float().T @ dy[a:b].float()))
                assert _relerr(W[gi], ref) < 5e-3
        else:
            assert torch.equal(W[gi], W0[gi]), f"group {gi}: weights of an unmasked group changed"
            assert torch.equal(dW[gi], dW_ref[gi]), f"group {gi}: gradient of an unmasked group differs"
    # the complement through the stand-alone kernel: afterwards every group is updated exactly once
    gg.sgd_step_groups(W, dW, lr, mask, want=False)
    W_all = W0.clone()
    gg.sgd_step(W_all, dW_ref, lr)
    torch.cuda.synchronize()
    assert torch.equal(W, W_all)


@pytest.mark.parametrize("pair_kernels", [False, True], ids=["1cta", "cta_pairs"])
def test_two_launches_share_one_ticket_counter(pair_kernels, cuda_device, monkeypatch):
    """One GEMM issued as two launches on two streams with a common ticket counter: every tile is
    computed exactly once, and the counter is clean afterwards (a third, ordinary dynamic launch
    that happens to get the same counter still computes everything)."""
    from moonep_b200.ops import grouped_gemm as gg
    monkeypatch.setenv("MOONEP_WGRAD_2CTA", "1" if pair_kernels else "0")
    rpg = [512, 0, 256, 1024, 128, 384]
    G, H, Hp = len(rpg), 512, 512
    cu, tot, rows, x, g = _setup(G, rpg, H, Hp, seed=3)
    wd = (torch.randn(G, Hp, H, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    dy = (torch.randn(rows, H, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    dgu = (torch.randn(rows, Hp, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    dA = torch.zeros(rows, Hp, dtype=torch.bfloat16, device="cuda")
    dW = torch.full((G, H, Hp), 3.0, device="cuda")
    side = torch.cuda.Stream()
    main = torch.cuda.current_stream()
    for _ in range(3):          # repeated use: the counter must come back to zero every time
        dA.zero_(); dW.fill_(3.0)
        side.wait_stream(main)
        tk1, tk2 = gg.Ticket(dA.device, 24), gg.Ticket(dA.device, 24)
        gg.dgrad(dy, wd, cu, dA, num_ctas=16, ticket=tk1)
        gg.wgrad(x, dgu, cu, dW, accumulate=True, num_ctas=16, ticket=tk2)
        with torch.cuda.stream(side):
            gg.dgrad(dy, wd, cu, dA, num_ctas=8, ticket=tk1)
            gg.wgrad(x, dgu, cu, dW, accumulate=True, num_ctas=8, ticket=tk2)
        main.wait_stream(side)
        torch.cuda.synchronize()
        gg.check_status()
        for gi, a, b in _group_slices(rpg):
            if a == b:
                assert (dW[gi] == 3.0).all()
                continue
            assert _relerr(dA[a:b], dy[a:b].float() @ wd[gi].float().T) < 1e-2, f"group {gi}: dgrad"
            assert _relerr(dW[gi], 3.0 + x[a:b].float().T @ dgu[a:b].float()) < 2e-3, f"group {gi}: wgrad (each tile once)"
    from moonep_b200.ops.grouped_gemm import _sched_cache
    assert int(_sched_cache[dA.device.index][0].abs().sum()) == 0, "ticket counters must be left at zero"


@pytest.mark.parametrize("split", [False, True], ids=["one_launch", "116+32_ctas_one_ticket"])
def test_benchmark_shape_against_fp32_on_sampled_tiles(split, cuda_device):
    """The shape the step benchmark runs (hidden 7168, inner 2048, 32 groups of uneven size, i.e. 112
    k-blocks per tile for gate/up and 32 for down, hundreds of tiles per CTA): every mode is checked
    against fp32 on sampled rows of sampled groups, once as a single launch and once as the two
    launches on one ticket counter that the layer uses beside a communication kernel."""
    from moonep_b200.ops import grouped_gemm as gg
    H, Hp, G = 7168, 2048, 32
    gen = torch.Generator(device="cuda").manual_seed(9)
    rpg = [128 * int(v) for v in torch.randint(0, 7, (G,), generator=torch.Generator().manual_seed(4))]
    rpg[3], rpg[17] = 0, 1152
    cu, tot, rows, x, _ = _setup(G, rpg, H, Hp, seed=9)
    wg = (torch.randn(G, H, Hp, device="cuda", generator=gen) * 0.02).to(torch.bfloat16)
    wu = (torch.randn(G, H, Hp, device="cuda", generator=gen) * 0.02).to(torch.bfloat16)
    wd = (torch.randn(G, Hp, H, device="cuda", generator=gen) * 0.02).to(torch.bfloat16)
    scale = torch.rand(rows, device="cuda", generator=gen) + 0.5
    sms = torch.cuda.get_device_properties(0).multi_processor_count

    def run(fn):
        """fn(num_ctas, ticket) launches one GEMM."""
        if not split:
            fn(None, None)
            return
        tk = gg.Ticket("cuda", sms)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        fn(sms - 32, tk)
        with torch.cuda.stream(side):
            fn(32, tk)
        torch.cuda.current_stream().wait_stream(side)

    act = torch.zeros(rows, Hp, dtype=torch.bfloat16, device="cuda")
    gu = torch.zeros(rows, 2 * Hp, dtype=torch.bfloat16, device="cuda")
    run(lambda n, tk: gg.gate_up(x, wg, wu, cu, act, gu, row_scale=scale, num_ctas=n, ticket=tk))
    y = torch.zeros(rows, H, dtype=torch.bfloat16, device="cuda")
    run(lambda n, tk: gg.down(act, wd, cu, y, num_ctas=n, ticket=tk))
    dA = torch.zeros(rows, Hp, dtype=torch.bfloat16, device="cuda")
    run(lambda n, tk: gg.dgrad(y, wd, cu, dA, num_ctas=n, ticket=tk))
    dx = torch.zeros(rows, H, dtype=torch.bfloat16, device="cuda")
    run(lambda n, tk: gg.dgrad_gate_up(gu, wg, wu, cu, dx, num_ctas=n, ticket=tk))
    dW = torch.zeros(G, H, Hp, device="cuda")
    run(lambda n, tk: gg.wgrad(x, act, cu, dW, accumulate=False, zero_empty_below=G, num_ctas=n, ticket=tk))
    torch.cuda.synchronize()
    gg.check_status()
    pick = torch.Generator().manual_seed(1)
    for gi, a, b in _group_slices(rpg):
        if a == b:
            assert (dW[gi] == 0).all()
            continue
        if gi % 3 and gi != 17:
            continue
        rsel = (a + torch.randperm(b - a, generator=pick)[:48]).cuda()       # rows from every 128-row tile region
        xf = x[rsel].float()
        gr, ur = xf @ wg[gi].float(), xf @ wu[gi].float()
        assert _relerr(gu[rsel, :Hp], gr) < 1e-2 and _relerr(gu[rsel, Hp:], ur) < 1e-2, f"group {gi}: pre-activations"
        assert _relerr(act[rsel], torch.nn.functional.silu(gr) * ur * scale[rsel, None]) < 1.5e-2, f"group {gi}: swiglu"
        assert _relerr(y[rsel], act[rsel].float() @ wd[gi].float()) < 1e-2, f"group {gi}: down"
        assert _relerr(dA[rsel], y[rsel].float() @ wd[gi].float().T) < 1e-2, f"group {gi}: dgrad"
        ref = gu[rsel, :Hp].float() @ wg[gi].float().T + gu[rsel, Hp:].float() @ wu[gi].float().T
        assert _relerr(dx[rsel], ref) < 1e-2, f"group {gi}: dgrad gate/up"
        csel = torch.randperm(Hp, generator=pick)[:64].cuda()
        wref = x[a:b].float().T @ act[a:b][:, csel].float()
        assert _relerr(dW[gi][:, csel], wref) < 3e-3, f"group {gi}: wgrad"
    assert (act[tot:] == 0).all() and (y[tot:] == 0).all(), "rows beyond cu_seqlens[-1] were written"
