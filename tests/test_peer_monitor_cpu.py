"""Host-side failure detection between steps (no GPU): real processes on a TCP store; one
rank leaves on purpose, one rank dies silently, and the healthy case."""
import os
import time

import torch.multiprocessing as mp


def _worker(rank, world, port, mode, q):
    from datetime import timedelta
    from torch.distributed import TCPStore
    from moonep_b200.utils.health import PeerMonitor, PeerLost
    store = TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=timedelta(seconds=30),
                     wait_for_workers=False)
    mon = PeerMonitor(store, rank, world)
    result = "completed"
    try:
        for step in range(6):
            if mode == "leaves" and rank == 2 and step == 3:
                mon.leave()                     # between steps, nothing in flight
                result = "left"
                break
            if mode == "dies" and rank == 1 and step == 2:
                result = "died"                 # stops publishing without a word
                break
            t0 = time.monotonic()
            mon.enter_step(step, timeout_s=1.5)
            assert time.monotonic() - t0 < 5.0
            time.sleep(0.02)                    # the "step"
    except PeerLost as e:
        result = ("lost", tuple(e.ranks), e.step, "left" if "left" in e.reason else "timeout")
    q.put((rank, result))
    store.set(f"done/{rank}", "1")
    if rank == 0:                               # the store lives in rank 0: outlive everyone's last access
        deadline = time.monotonic() + 20
        while time.monotonic() < deadline and not store.check([f"done/{r}" for r in range(world)]):
            time.sleep(0.05)
        time.sleep(0.2)


def _run(world, mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29950 + (os.getpid() % 40) + {"ok": 0, "leaves": 50, "dies": 100}[mode]
    procs = [ctx.Process(target=_worker, args=(r, world, port, mode, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = dict(q.get(timeout=60) for _ in range(world))
    for p in procs:
        p.join(30)
        assert p.exitcode == 0, f"worker exited with {p.exitcode}"
    return out


def test_all_ranks_healthy():
    assert _run(3, "ok") == {0: "completed", 1: "completed", 2: "completed"}


def test_rank_that_leaves_is_reported_before_the_next_step():
    res = _run(3, "leaves")
    assert res[2] == "left"
    for r in (0, 1):
        assert res[r] == ("lost", (2,), 3, "left"), res


def test_rank_that_dies_is_reported_after_the_timeout():
    res = _run(3, "dies")
    assert res[1] == "died"
    for r in (0, 2):
        assert res[r] == ("lost", (1,), 2, "timeout"), res
