"""A rank leaves the EP group between steps; its peers learn of it on the host.

Run:  torchrun --nproc-per-node N --master-addr 127.0.0.1 --master-port P tests/dist_peer_leave.py
Every rank runs dispatch + combine steps through the public API.  Before each step it calls
``PeerMonitor.enter_step``.  After three steps the last rank stops taking part: it waits for
its own work to finish, publishes that it leaves and skips the remaining steps (its process
and its memory stay until the common teardown, so no peer ever touches unmapped memory).  The
others must get ``PeerLost`` for exactly that rank at step 3, on the host, before launching
anything that would wait for it -- no device-side wait runs out, no status word is set.
Nothing here faults, traps or hangs a GPU.
"""
import json
import os
import sys
from datetime import timedelta

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from moonep_b200 import Buffer, routing  # noqa: E402
from moonep_b200.utils import PeerLost, PeerMonitor  # noqa: E402


def main():
    dist.init_process_group("nccl")
    rank, R = dist.get_rank(), dist.get_world_size()
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    store = dist.TCPStore("127.0.0.1", int(os.environ["MASTER_PORT"]) + 37, R, is_master=(rank == 0),
                          timeout=timedelta(seconds=60), wait_for_workers=False)
    S, H, K, epn, pad = 64, 256, 2, 4, 16
    E = R * epn
    buf = Buffer(S, H, K, E, R, num_sms=2, token_padding=pad)
    mon = PeerMonitor(store, rank, R)
    topk, tpe = routing.lognormal_topk(S, K, E, R, 1.0, 5, rank)
    topk, tpe = topk.cuda(), tpe.cuda()
    hidden = ((torch.arange(S * H) % 13) - 6).reshape(S, H).to(torch.bfloat16).cuda()    # small integers: sums are exact
    leaver, leave_at = R - 1, 3
    steps_done, status, wrong = 0, "completed", 0
    try:
        for step in range(6):
            if rank == leaver and step == leave_at:
                torch.cuda.synchronize()            # nothing of mine is in flight
                mon.leave()
                status = "left"
                break
            mon.enter_step(step, timeout_s=20.0)
            h, _, _, plan = buf.dispatch(hidden, None, topk, tpe)
            out, _, _ = buf.combine(plan=plan, hidden_nvsh=h)
            torch.cuda.synchronize()
            buf.check()                             # no device-side wait ran out
            wrong += int((out.float() != hidden.float() * K).sum())
            steps_done += 1
    except PeerLost as exc:
        status = f"lost:{','.join(map(str, exc.ranks))}@{exc.step}"
    torch.cuda.synchronize()
    print("RESULT " + json.dumps({"rank": rank, "status": status, "steps": steps_done, "wrong": wrong}), flush=True)
    # common teardown: every rank, the one that left included, releases its memory together
    buf.destroy()
    store.set(f"bye/{rank}", "1")
    if rank == 0:
        store.wait([f"bye/{r}" for r in range(R)], timedelta(seconds=30))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
