"""The allocation-free planner entry point (csrc/mep_noalloc.h), called through its exported C
symbol, must produce exactly what the regular planner produces -- on two calls in a row, since
both share one built-in work space that keeps the previous call's contents.

It serves callers that cannot allocate device memory when they need a plan (allocator
callbacks, real-time loops that must avoid cudaMalloc's implicit synchronisation, processes
with a fixed memory budget). Collected last on purpose: a run that stops at the first failure
has then already exercised every other test.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _regular_plan(S, K, E, pad, topk, tpe):
    from moonep_b200 import engine
    from moonep_b200.sim.local_cluster import LocalCluster
    cl = LocalCluster(S, 64, K, E, 1, num_sms=4, token_padding=pad)
    st = cl._states
    plan, cu = engine.allocate_plan(st[0])
    engine.launch_planning(st, [topk], [tpe], [plan], [cu])
    torch.cuda.synchronize()
    cl.check()
    return plan, cu


def _noalloc_plan(lib, S, K, E, pad, topk, tpe, check_free=False):
    i32 = dict(dtype=torch.int32, device="cuda")
    dst = torch.full((S * K,), 123456, **i32)
    cu = torch.full((2 * E,), 123456, **i32)
    zfr = torch.full((2 * E, 2), 123456, **i32)
    etc = torch.full((E,), 123456, **i32)
    stats = torch.full((2,), 123456, **i32)
    before = torch.cuda.memory_allocated()
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    rc = lib.mep_plan_single_rank_noalloc(
        C.c_void_p(topk.data_ptr()), C.c_void_p(tpe.data_ptr()), S, K, E, pad,
        C.c_void_p(dst.data_ptr()), C.c_void_p(cu.data_ptr()), C.c_void_p(zfr.data_ptr()),
        C.c_void_p(etc.data_ptr()), C.c_void_p(stats.data_ptr()),
        C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, lib.mep_last_error().decode()
    assert torch.cuda.memory_allocated() == before
    torch.cuda.synchronize()
    # the driver's own count of free device memory sees raw cudaMalloc calls as well, which torch's
    # counter does not; only checked once the kernel's code is resident (the first call of a process
    # loads it, which takes device memory)
    if check_free:
        assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the amount of free device memory"
    return dst, cu, zfr, etc, stats


@pytest.mark.parametrize("first,second", [((300, 6, 40, 16), (64, 4, 8, 128)), ((1000, 8, 256, 128), (1000, 8, 256, 128))])
def test_noalloc_planner_matches_regular(first, second, cuda_device):
    from moonep_b200 import _native
    lib = _native.load()
    lib.mep_plan_single_rank_noalloc.restype = C.c_int
    for call, (S, K, E, pad) in enumerate((first, second)):
        g = torch.Generator(device="cuda").manual_seed(17 + call)
        topk = torch.randint(0, E, (S, K), dtype=torch.int32, device="cuda", generator=g)
        tpe = torch.zeros(E, dtype=torch.int32, device="cuda")
        tpe.scatter_add_(0, topk.reshape(-1).long(), torch.ones(S * K, dtype=torch.int32, device="cuda"))
        dst, cu, zfr, etc, stats = _noalloc_plan(lib, S, K, E, pad, topk.reshape(-1).contiguous(), tpe, check_free=call > 0)
        plan, cu_ref = _regular_plan(S, K, E, pad, topk.reshape(-1).contiguous(), tpe)
        assert torch.equal(dst, plan.dst), f"call {call}: dst differs"
        assert torch.equal(cu, cu_ref), f"call {call}: cu_seqlens differs"
        assert torch.equal(zfr, plan.zero_fill_ranges), f"call {call}: zero_fill_ranges differs"
        assert torch.equal(etc.view(1, E), plan.experts_to_copy), f"call {call}: experts_to_copy differs"
        assert torch.equal(stats, plan.remote_stats), f"call {call}: remote_stats differs"


def test_noalloc_rejects_oversize(cuda_device):
    from moonep_b200 import _native
    lib = _native.load()
    lib.mep_plan_single_rank_noalloc.restype = C.c_int
    t = torch.zeros(8, dtype=torch.int32, device="cuda")
    p = C.c_void_p(t.data_ptr())
    assert lib.mep_plan_single_rank_noalloc(p, p, 70000, 1, 8, 1, p, p, p, p, p, None) == -1
    assert b"exceeds the built-in work space" in lib.mep_last_error()
    assert lib.mep_plan_single_rank_noalloc(p, p, 8, 1, 2048, 1, p, p, p, p, p, None) == -1
    assert b"max 1024 experts" in lib.mep_last_error()


def test_noalloc_rejects_a_capturing_stream(cuda_device):
    """Under stream capture the copy of the rank context would be replayed from a dead stack frame, so
    the entry point refuses: nothing is recorded and the capture stays valid."""
    from moonep_b200 import _native
    lib = _native.load()
    lib.mep_plan_single_rank_noalloc.restype = C.c_int
    S, K, E, pad = 64, 2, 8, 16
    topk = torch.randint(0, E, (S * K,), dtype=torch.int32, device="cuda")
    tpe = torch.bincount(topk.long(), minlength=E).to(torch.int32)
    outs = [torch.zeros(n, dtype=torch.int32, device="cuda") for n in (S * K, 2 * E, 4 * E, E, 2)]
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        graph.capture_begin()
        try:
            rc = lib.mep_plan_single_rank_noalloc(C.c_void_p(topk.data_ptr()), C.c_void_p(tpe.data_ptr()), S, K, E, pad,
                                                  *[C.c_void_p(o.data_ptr()) for o in outs], C.c_void_p(side.cuda_stream))
            msg = lib.mep_last_error()
        finally:
            graph.capture_end()
    assert rc == -1 and b"being captured" in msg
    torch.cuda.synchronize()
