"""Python front end of the tcgen05 grouped expert GEMM (csrc/device/grouped_gemm.cu) and its
element-wise companions (csrc/device/swiglu.cu).

Conventions: ``x`` is the dispatched token matrix ``[NvS, in]`` in VM-group order;
``cu_seqlens[G]`` holds each group's padded end row (multiples of 128); weights are
``[G, in, out]`` bf16 (G = 2*epn: local experts then prefetch slots).  All functions launch
on the current stream and fail loudly if the native library is missing.

The reference ships no GEMM: it hands ``hidden_nvsh``, ``cu_seqlens`` and the ``[2*epn, H, H']``
compute view to the integrating framework's grouped GEMM (README.md:45, 54 of the reference;
moonep/dispatch.py:454 names DeepGEMM as the consumer).  This module is that consumer.
"""

from __future__ import annotations

import ctypes as C
import os

import torch

from .. import _native

GATE_UP, DOWN, DGRAD, DGRAD_GU, WGRAD = range(5)
_status_cache: dict = {}
_sm_cache: dict = {}


class GemmArgs(C.Structure):
    _fields_ = [("cu_seqlens", C.c_void_p), ("G", C.c_int32), ("N", C.c_int32), ("K", C.c_int32),
                ("M_w", C.c_int32), ("b_group_rows", C.c_int32), ("accumulate", C.c_int32),
                ("g_begin", C.c_int32), ("g_end", C.c_int32), ("zero_empty_below", C.c_int32), ("reserved0", C.c_int32),
                ("out", C.c_void_p), ("out2", C.c_void_p), ("row_scale", C.c_void_p), ("ldo", C.c_int64),
                ("status", C.c_void_p), ("budget_ns", C.c_uint64), ("sched", C.c_void_p),
                ("push_info", C.c_void_p), ("push_base", C.c_void_p), ("push_wbase", C.c_void_p),
                ("push_wsrc", C.c_void_p), ("push_stride", C.c_uint64),
                ("tile_done", C.c_void_p), ("tile_epoch", C.c_void_p), ("status_host", C.c_void_p),
                ("group_flags", C.c_void_p), ("group_epoch", C.c_void_p),
                ("push_rows", C.c_int32), ("push_ranks", C.c_int32), ("group_first", C.c_int32), ("sched_ctas", C.c_int32),
                ("upd_w", C.c_void_p), ("upd_mask", C.c_void_p), ("upd_lr", C.c_float), ("reserved1", C.c_int32)]


class PushTarget:
    """Where a "push" epilogue sends its rows (see ``Buffer.push_target``): ``info[r]`` names the
    source rank and receive row of output row ``r``; ``base`` / ``wbase`` are the addresses of rank
    0's receive areas, ``stride`` the distance to the next rank's, ``rows`` = S*K."""

    def __init__(self, info, base, wbase, stride, rows, ranks):
        self.info, self.base, self.wbase, self.stride, self.rows, self.ranks = info, base, wbase, stride, rows, ranks


def _dev_index(device) -> int:
    idx = torch.device(device).index
    return torch.cuda.current_device() if idx is None else idx


def _status(device) -> torch.Tensor:
    key = _dev_index(device)
    if key not in _status_cache:
        _status_cache[key] = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", key))
    return _status_cache[key]


_status_host_cache: dict = {}


def _status_host(device) -> torch.Tensor:
    """Pinned host word the GEMM kernels mirror their failure code into (see ``failed``)."""
    key = _dev_index(device)
    if key not in _status_host_cache:
        _status_host_cache[key] = torch.zeros(1, dtype=torch.int32).pin_memory()
    return _status_host_cache[key]


def failed(device="cuda") -> bool:
    """True once a grouped GEMM on ``device`` has given up a wait.  Reads host memory only (no
    synchronisation); ``check_status`` gives the details and clears the state."""
    t = _status_host_cache.get(_dev_index(device))
    return t is not None and int(t[0]) != 0


_SCHED_SLOTS = 64
_sched_cache: dict = {}


class Ticket:
    """A ticket counter that several launches of ONE grouped GEMM share: the launches (e.g. one on
    the compute stream beside a communication kernel, a second one behind that kernel on its
    stream) then split the GEMM's tiles between them dynamically.  ``total_ctas`` is the sum of
    the launches' CTA counts; every launch must be issued, and the counter is clean again once the
    last of them has finished."""

    def __init__(self, device, total_ctas: int):
        self.ptr = _sched(device, True, force=True)
        self.total_ctas = int(total_ctas)


def _sched(device, dynamic: bool, force: bool = False) -> int:
    """Ticket counter for one launch with the dynamic tile scheduler, or 0 for the static tile
    order.  ``dynamic`` is the caller's wish (set for GEMMs that run beside a communication kernel,
    where CTAs start late); ``MOONEP_GEMM_DYNAMIC=1`` / ``=0`` forces it on / off for every launch.
    Counters are handed out round-robin from a per-device pool so that GEMMs running concurrently
    on different streams never share one; each kernel leaves its counter at zero."""
    env = os.environ.get("MOONEP_GEMM_DYNAMIC")
    if env is not None and not force:
        dynamic = env == "1"
    if not dynamic:
        return 0
    key = _dev_index(device)
    ent = _sched_cache.get(key)
    if ent is None:
        ent = _sched_cache[key] = [torch.zeros(2 * _SCHED_SLOTS, dtype=torch.int32, device=torch.device("cuda", key)), 0]
    ent[1] = (ent[1] + 1) % _SCHED_SLOTS
    return ent[0].data_ptr() + 8 * ent[1]


def _num_sms(device) -> int:
    key = _dev_index(device)
    if key not in _sm_cache:
        _sm_cache[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return _sm_cache[key]


def check_status(device="cuda") -> None:
    """Synchronise and raise if a GEMM pipeline wait expired."""
    st = _status(device)
    v = st.cpu().tolist()
    if v[0] != 0:
        st.zero_()
        _status_host(device).zero_()
        ent = _sched_cache.get(_dev_index(device))
        if ent is not None:
            ent[0].zero_()
        raise RuntimeError(f"grouped GEMM aborted: code {v[0]} at site {v[1]}, CTA {v[2]}, tile {v[3]}")


def _launch(mode, a, b0, b1, cu, *, N, K=0, M_w=0, b_group_rows=0, out, out2=None, row_scale=None, ldo=0,
            accumulate=False, zero_empty_below=0, a_cols=None, b_rows=None, b_cols=None, b_ld=None, groups=None, num_ctas=None,
            dynamic=False, ticket=None, push=None, push_w=None, ready=None, slots=None):
    lib = _native.load()
    assert a.dtype == torch.bfloat16 and b0.dtype == torch.bfloat16
    assert cu.dtype == torch.int32 and cu.is_contiguous()
    G = cu.numel()
    g0, g1 = (0, G) if groups is None else groups
    args = GemmArgs()
    args.cu_seqlens = cu.data_ptr()
    args.G, args.N, args.K, args.M_w = G, N, K, M_w
    args.b_group_rows, args.accumulate = b_group_rows, 1 if accumulate else 0
    args.g_begin, args.g_end = g0, g1
    args.zero_empty_below = zero_empty_below
    args.out, args.out2 = out.data_ptr(), _native.ptr(out2)
    args.row_scale, args.ldo = _native.ptr(row_scale), ldo
    args.status = _status(a.device).data_ptr()
    args.status_host = _status_host(a.device).data_ptr()
    from ..engine import wait_budget_ns
    args.budget_ns = wait_budget_ns()
    if ticket is not None:
        args.sched, args.sched_ctas = ticket.ptr, ticket.total_ctas
    else:
        args.sched = _sched(a.device, dynamic)
    if ready is not None:
        assert mode in (GATE_UP, DGRAD), "ready flags gate the GEMMs that read the dispatched rows"
        args.tile_done, args.tile_epoch = ready.done_ptr, ready.epoch_ptr
    if slots is not None:
        args.group_flags, args.group_epoch, args.group_first = slots.flags_ptr, slots.epoch_ptr, slots.first
    if push is not None:
        assert mode in (DOWN, DGRAD, DGRAD_GU) and push.info.dtype == torch.int32 and push.info.numel() >= a.shape[0]
        args.push_info, args.push_base, args.push_stride = push.info.data_ptr(), push.base, push.stride
        args.push_rows, args.push_ranks = push.rows, push.ranks
        if push_w is not None:
            assert push_w.dtype == torch.float32 and push_w.numel() >= a.shape[0]
            args.push_wsrc, args.push_wbase = push_w.data_ptr(), push.wbase
    a_rows = a.shape[0]
    a_ld = a.stride(0)
    a_cols = a.shape[1] if a_cols is None else a_cols
    fn = lib.mep_grouped_gemm
    if mode != WGRAD and push is None and ready is None and slots is None and os.environ.get("MOONEP_GEMM_2CTA", "0") == "1":
        fn = lib.mep_grouped_gemm_2cta      # CTA-pair kernels (tcgen05 cta_group::2), 256-token tiles
    rc = fn(mode, C.c_void_p(a.data_ptr()), C.c_int64(a_rows), C.c_int64(a_cols), C.c_int64(a_ld),
                              C.c_void_p(b0.data_ptr()), C.c_void_p(_native.ptr(b1)), C.c_int64(b_rows),
                              C.c_int64(b_cols), C.c_int64(b_ld), C.byref(args),
                              num_ctas or _num_sms(a.device), _native.cur_stream())
    _native.check(rc, "grouped_gemm")


def _w2d(w):
    assert w.dim() == 3 and w.is_contiguous(), "weights must be contiguous [G, in, out]"
    return w.shape[0] * w.shape[1], w.shape[2]


def gate_up(x, wg, wu, cu, act_out, gu_out=None, row_scale=None, groups=None, num_ctas=None, dynamic=False, ticket=None,
            ready=None, slots=None):
    """``act_out[r] = row_scale[r] * silu(x[r] Wg[g]) * (x[r] Wu[g])``; optionally stores the
    pre-activations ``gu_out = [x Wg | x Wu]`` (``[NvS, 2*out]``) for the backward pass.
    ``ready`` (a ``TileReady`` from ``Buffer.dispatch_ready``): ``x`` is still being filled by that
    dispatch; every 128-row tile is loaded only once its flag says it is complete.  Launch with
    ``num_ctas <= ready.free_sms`` while the dispatch kernel may still be running.
    ``slots`` (a ``SlotReady`` from ``Buffer.slot_ready``): the weights of the groups ``>= slots.first`` are
    prefetched experts that may still be on their way; each such group is loaded once its slot is complete."""
    G, K, N = wg.shape
    assert wu.shape == wg.shape and x.shape[1] == K and N % 128 == 0 and K % 64 == 0
    rows, cols = _w2d(wg)
    _launch(GATE_UP, x, wg, wu, cu, N=N, K=K, b_group_rows=K, out=act_out, out2=gu_out, row_scale=row_scale,
            ldo=act_out.stride(0), b_rows=rows, b_cols=cols, b_ld=cols, groups=groups, num_ctas=num_ctas, dynamic=dynamic, ticket=ticket,
            ready=ready, slots=slots)


def down(act, wd, cu, out, row_scale=None, groups=None, num_ctas=None, dynamic=False, ticket=None, push=None):
    """``out[r] = row_scale[r] * (act[r] Wd[g])`` with ``Wd [G, inner, hidden]``.  With ``push`` (a
    ``PushTarget``) the rows are not written to ``out`` but sent to the ranks their tokens came from."""
    G, K, N = wd.shape
    assert act.shape[1] == K and N % 256 == 0 and K % 64 == 0
    rows, cols = _w2d(wd)
    _launch(DOWN, act, wd, None, cu, N=N, K=K, b_group_rows=K, out=out, row_scale=row_scale, ldo=out.stride(0),
            b_rows=rows, b_cols=cols, b_ld=cols, groups=groups, num_ctas=num_ctas, dynamic=dynamic, ticket=ticket, push=push)


def dgrad(dy, w, cu, out, groups=None, num_ctas=None, dynamic=False, ticket=None, ready=None, slots=None):
    """``out[r] = dy[r] W[g]^T`` with ``W [G, in, out]`` -> ``out [NvS, in]``.  ``ready`` / ``slots``: as in ``gate_up``."""
    G, N, K = w.shape
    assert dy.shape[1] == K and N % 256 == 0 and K % 64 == 0
    rows, cols = _w2d(w)
    _launch(DGRAD, dy, w, None, cu, N=N, K=K, b_group_rows=N, out=out, ldo=out.stride(0),
            b_rows=rows, b_cols=cols, b_ld=cols, groups=groups, num_ctas=num_ctas, dynamic=dynamic, ticket=ticket, ready=ready,
            slots=slots)


def dgrad_gate_up(dgu, wg, wu, cu, out, groups=None, num_ctas=None, dynamic=False, ticket=None, push=None, push_w=None):
    """``out[r] = dG[r] Wg[g]^T + dU[r] Wu[g]^T`` with ``dgu = [dG | dU]`` (``[NvS, 2*inner]``).  With
    ``push`` the rows (and ``push_w[r]``, e.g. the route-weight grads) go to their source ranks."""
    G, N, Kh = wg.shape
    assert dgu.shape[1] == 2 * Kh and N % 256 == 0 and Kh % 64 == 0
    rows, cols = _w2d(wg)
    _launch(DGRAD_GU, dgu, wg, wu, cu, N=N, K=2 * Kh, b_group_rows=N, out=out, ldo=out.stride(0),
            b_rows=rows, b_cols=cols, b_ld=cols, groups=groups, num_ctas=num_ctas, dynamic=dynamic, ticket=ticket,
            push=push, push_w=push_w)


def wgrad_update_supported(M: int, N: int) -> bool:
    """Whether ``wgrad(update=...)`` exists for ``[M, N]`` weight matrices (the CTA-pair kernel carries it)."""
    return M % 256 == 0 and N % 256 == 0 and os.environ.get("MOONEP_WGRAD_2CTA", "1") != "0"


def wgrad(x, dy, cu, out, accumulate=False, zero_empty_below=0, groups=None, num_ctas=None, dynamic=False, ticket=None,
          update=None):
    """``out[g] (+)= x_g^T dy_g`` in fp32; ``out [G, in, out_dim]``.  ``dy`` may be a column slice
    of a wider matrix (row pitch = ``dy.stride(0)``).  Groups without rows are left untouched,
    except that with ``accumulate=False`` empty groups ``g < zero_empty_below`` are zeroed (local
    experts that received no token must end with a zero gradient).

    ``update=(weights, lr, mask)``: optimizer in the epilogue.  For every group with ``mask[g] != 0``
    (int32 ``[G]`` on the device) the gradient is not written; ``weights[g]`` (bf16, same shape as ``out``)
    becomes ``weights[g] - lr * dW`` instead, bit for bit what ``sgd_step`` computes from a stored gradient.
    Groups with ``mask[g] == 0`` are written to ``out`` as usual.  Needs weight shapes that are multiples
    of 256 (the CTA-pair kernel)."""
    G, M, N = out.shape
    assert out.dtype == torch.float32 and out.is_contiguous()
    assert x.shape[1] == M and dy.shape[1] == N and M % 128 == 0 and N % 256 == 0
    assert dy.stride(1) == 1 and x.stride(1) == 1
    if M % 256 == 0 and os.environ.get("MOONEP_WGRAD_2CTA", "1") != "0":
        # CTA-pair kernel (tcgen05 cta_group::2): a third less operand traffic per SM
        lib = _native.load()
        G0, G1 = (0, G) if groups is None else groups
        args = GemmArgs()
        args.cu_seqlens = cu.data_ptr()
        args.G, args.N, args.K, args.M_w = G, N, 0, M
        args.accumulate, args.g_begin, args.g_end = (1 if accumulate else 0), G0, G1
        args.zero_empty_below = zero_empty_below
        args.out = out.data_ptr()
        args.status = _status(x.device).data_ptr()
        args.status_host = _status_host(x.device).data_ptr()
        from ..engine import wait_budget_ns
        args.budget_ns = wait_budget_ns()
        if ticket is not None:
            args.sched, args.sched_ctas = ticket.ptr, ticket.total_ctas
        else:
            args.sched = _sched(x.device, dynamic)
        if update is not None:
            w, lr, mask = update
            assert w.dtype == torch.bfloat16 and tuple(w.shape) == tuple(out.shape) and w.is_contiguous()
            assert mask.dtype == torch.int32 and mask.numel() == G and mask.is_cuda
            args.upd_w, args.upd_mask, args.upd_lr = w.data_ptr(), mask.data_ptr(), float(lr)
        rc = lib.mep_grouped_wgrad_2cta(C.c_void_p(x.data_ptr()), C.c_int64(x.shape[0]), C.c_int64(x.stride(0)),
                                        C.c_void_p(dy.data_ptr()), C.c_int64(dy.stride(0)), C.byref(args),
                                        num_ctas or _num_sms(x.device), _native.cur_stream())
        _native.check(rc, "grouped_wgrad_2cta")
        return
    assert update is None, "wgrad(update=...) needs weight shapes that are multiples of 256"
    _launch(WGRAD, x, dy, None, cu, N=N, M_w=M, out=out, accumulate=accumulate, zero_empty_below=zero_empty_below,
            b_rows=dy.shape[0], b_cols=N, b_ld=dy.stride(0), groups=groups, num_ctas=num_ctas, dynamic=dynamic, ticket=ticket)


def swiglu_bwd(dA, gu, w, dgu, dw, cu, num_blocks=None):
    """Backward of ``act = w * silu(g) * u``: fills ``dgu = [dG | dU]`` and ``dw[row]``."""
    lib = _native.load()
    Hp = dA.shape[1]
    nb = num_blocks or 4 * _num_sms(dA.device)
    _native.check(lib.mep_swiglu_bwd(C.c_void_p(dA.data_ptr()), C.c_void_p(gu.data_ptr()), C.c_void_p(_native.ptr(w)),
                                     C.c_void_p(dgu.data_ptr()), C.c_void_p(_native.ptr(dw)), C.c_void_p(cu.data_ptr()),
                                     cu.numel(), Hp, nb, _native.cur_stream()), "swiglu_bwd")


def sgd_step_groups(p, g, lr, mask, want: bool, num_blocks=None):
    """``sgd_step`` for the groups ``i`` of ``p [G, ...]`` with ``(mask[i] != 0) == want`` only (``mask``: int32
    ``[>= G]`` on the device): the complement of what ``wgrad(update=...)`` has already updated."""
    lib = _native.load()
    assert p.dtype == torch.bfloat16 and g.dtype == torch.float32 and p.shape == g.shape
    assert p.is_contiguous() and g.is_contiguous() and mask.dtype == torch.int32 and mask.numel() >= p.shape[0]
    nb = num_blocks or 2 * _num_sms(p.device)
    _native.check(lib.mep_sgd_step_groups(C.c_void_p(p.data_ptr()), C.c_void_p(g.data_ptr()), C.c_float(lr),
                                          C.c_int64(p[0].numel()), p.shape[0], C.c_void_p(mask.data_ptr()), 1 if want else 0,
                                          nb, _native.cur_stream()), "sgd_step_groups")


def sgd_step(p, g, lr, num_blocks=None):
    lib = _native.load()
    assert p.dtype == torch.bfloat16 and g.dtype == torch.float32 and p.numel() == g.numel()
    assert p.is_contiguous() and g.is_contiguous()
    nb = num_blocks or 8 * _num_sms(p.device)
    _native.check(lib.mep_sgd_step(C.c_void_p(p.data_ptr()), C.c_void_p(g.data_ptr()), C.c_float(lr),
                                   C.c_int64(p.numel()), nb, _native.cur_stream()), "sgd_step")
