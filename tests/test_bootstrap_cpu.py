"""CPU tests of the bootstrap path and of host-side failure handling (no GPU):
descriptor exchange over unix sockets between real processes (gloo group), a rank that never
sends, a closed/invalid descriptor, and the host model of the epoch barrier."""
import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from moonep_b200.sim.barrier_model import EpochBarrierModel


def _worker(rank, world, port, mode, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from moonep_b200.parallel import symm
    try:
        if mode == "ok":
            # every rank shares the read end of its own pipe; afterwards rank r writes one byte into
            # its pipe and reads it back through the descriptor it received for ITSELF, and checks
            # that every received descriptor is a live pipe
            rfd, wfd = os.pipe()
            fds = symm.exchange_fds(rfd, None)
            os.write(wfd, bytes([65 + rank]))
            dist.barrier()
            got = os.read(fds[rank], 1)
            import stat
            ok = len(fds) == world and all(stat.S_ISFIFO(os.fstat(fd).st_mode) for fd in fds) and got == bytes([65 + rank])
            for fd in fds:
                os.close(fd)
            os.close(rfd); os.close(wfd)
            q.put((rank, "ok" if ok else "bad"))
        elif mode == "subgroups":
            # two disjoint EP groups of two ranks inside one job (what ``Buffer(group=...)`` relies
            # on): each group exchanges among its own members only, addressed by group rank
            groups = [dist.new_group([0, 1]), dist.new_group([2, 3])]
            mine = groups[rank // 2]
            rfd, wfd = os.pipe()
            fds = symm.exchange_fds(rfd, mine)
            os.write(wfd, bytes([65 + rank]) * 2)      # one byte for me, one for my partner
            dist.barrier()
            got = os.read(fds[dist.get_rank(mine)], 1)
            ok = len(fds) == 2 and got == bytes([65 + rank])
            # the partner's descriptor must be the partner's pipe: it holds the partner's byte
            other = os.read(fds[1 - dist.get_rank(mine)], 1)
            ok = ok and other == bytes([65 + (rank ^ 1)])
            for fd in fds:
                os.close(fd)
            os.close(rfd); os.close(wfd)
            q.put((rank, "ok" if ok else "bad"))
        elif mode == "silent_rank":
            # the last rank skips the send: the others must time out with a clean error
            symm.IPC_TIMEOUT_MS = 500
            from moonep_b200 import _native
            import ctypes as C
            lib = _native.load()
            box = [tempfile.mkdtemp(prefix="mep_t_") if rank == 0 else None]
            dist.broadcast_object_list(box, src=0)
            ep = C.c_void_p()
            _native.check(lib.mep_ipc_open(box[0].encode(), rank, world, C.byref(ep)), "open")
            dist.barrier()
            rfd, wfd = os.pipe()
            if rank != world - 1:
                _native.check(lib.mep_ipc_send_all(ep, rfd), "send")
            fds = (C.c_int * world)()
            rc = lib.mep_ipc_recv_all(ep, fds, 500)
            msg = lib.mep_last_error().decode()
            lib.mep_ipc_close(ep)
            dist.barrier()
            q.put((rank, "timeout" if rc != 0 and "timed out" in msg and all(f == -1 for f in fds) else f"unexpected rc={rc} {msg}"))
        elif mode == "bad_fd":
            from moonep_b200 import _native
            import ctypes as C
            lib = _native.load()
            box = [tempfile.mkdtemp(prefix="mep_t_") if rank == 0 else None]
            dist.broadcast_object_list(box, src=0)
            ep = C.c_void_p()
            _native.check(lib.mep_ipc_open(box[0].encode(), rank, world, C.byref(ep)), "open")
            dist.barrier()
            rc = lib.mep_ipc_send_all(ep, 987654)          # not an open descriptor
            msg = lib.mep_last_error().decode()
            lib.mep_ipc_close(ep)
            dist.barrier()
            q.put((rank, "rejected" if rc != 0 and "sendmsg" in msg else f"unexpected rc={rc}"))
    finally:
        dist.destroy_process_group()


def _run(world, mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + (os.getpid() % 300)
    procs = [ctx.Process(target=_worker, args=(r, world, port, mode, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0, f"worker exited with {p.exitcode}"
    return dict(q.get(timeout=5) for _ in range(world))


def test_fd_exchange_between_processes():
    res = _run(3, "ok")
    assert res == {0: "ok", 1: "ok", 2: "ok"}


def test_fd_exchange_inside_subgroups():
    res = _run(4, "subgroups")
    assert res == {0: "ok", 1: "ok", 2: "ok", 3: "ok"}


def test_rank_that_never_sends_times_out_cleanly():
    res = _run(2, "silent_rank")
    assert all(v == "timeout" for v in res.values()), res


def test_invalid_descriptor_is_rejected():
    res = _run(2, "bad_fd")
    assert all(v == "rejected" for v in res.values()), res


def test_handle_type_env(monkeypatch):
    from moonep_b200.parallel import symm
    monkeypatch.setenv("MOONEP_MEM_HANDLE_TYPE", "bogus")
    with pytest.raises(ValueError, match="auto|fabric|fd"):
        symm.resolve_handle_kind(0, None)
    monkeypatch.setenv("MOONEP_MEM_HANDLE_TYPE", "fd")
    assert symm.resolve_handle_kind(0, None) == symm.HANDLE_FD


def test_barrier_model_detects_missing_rank():
    b = EpochBarrierModel(4)
    for r in range(4):
        b.arrive(r)
    assert all(b.wait(r).ok for r in range(4))
    # next barrier: rank 2 never arrives
    for r in (0, 1, 3):
        b.arrive(r)
    st = b.wait(0, polls=8)
    assert not st.ok and st.peer == 2 and st.expected == 2 and st.observed == 1
    # a dropped arrival (rank 1's store to rank 3 lost)
    b.reset()
    for r in range(4):
        b.arrive(r, drop_to={3} if r == 1 else None)
    assert b.wait(0).ok and not b.wait(3).ok and b.wait(3).peer == 1
    # late arrival repairs it: epochs are monotone, nothing to reset
    b.flags[3][1] = b.epoch[1]
    assert b.wait(3).ok


def test_native_library_loads_without_gpu():
    from moonep_b200 import _native
    lib = _native.load()
    assert lib.mep_abi_version() >= 1
    assert isinstance(lib.mep_launch_count(), int)


def test_ctypes_mirrors_match_the_compiled_struct_sizes():
    """Every argument struct that Python fills through ctypes has the size the compiler gave its
    C++ definition (the library exports sizeof for each); a field added on one side only shows up
    here instead of as a corrupted kernel argument."""
    import ctypes as C
    from moonep_b200 import _native
    from moonep_b200.ops.grouped_gemm import GemmArgs
    lib = _native.load()
    mirrors = {
        "MepRankCtx": _native.MepRankCtx, "MepStatus": _native.MepStatus, "PlanArgs": _native.PlanArgs,
        "DispatchArgs": _native.DispatchArgs, "DupFinalizeArgs": _native.DupFinalizeArgs,
        "DupArgs": _native.DupArgs, "DupFreshArgs": _native.DupArgs, "CombineArgs": _native.CombineArgs,
        "PushReduceArgs": _native.PushReduceArgs, "PrefetchArgs": _native.PrefetchArgs,
        "GradReduceArgs": _native.GradReduceArgs, "GemmArgs": GemmArgs, "SendOrderArgs": _native.SendOrderArgs,
    }
    for name, cls in mirrors.items():
        native = getattr(lib, f"mep_sizeof_{name}")()
        assert C.sizeof(cls) == native, f"{name}: ctypes {C.sizeof(cls)} bytes, compiled {native} bytes"
