"""``bench.py --verify-plans``: on N >= 2 GPUs feed IDENTICAL routing tables to this package's Buffer and
to the unmodified reference package's Buffer (installed under ``baseline/_ref``) and compare what the
two planners produce on the device: ``dst`` (with its duplicate sign encoding), ``cu_seqlens``,
``experts_to_copy``, ``zero_fill_ranges``, ``remote_stats`` element by element, the duplicate groups as
sets (their order is unspecified in both implementations), and the dispatched rows themselves.  One JSON
line on rank 0: ``{"verify_plans": "pass" | "fail", ...}``.

The two packages are used one after the other in one process; nothing of one is handed to the other
except plain tensors of routing tables and results copied to the host.
"""
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
SKEWS = (0.0, 1.0, 3.0)


def _dups(groups, loffs, counts):
    g, l, c = groups.cpu().numpy(), loffs.cpu().numpy(), counts.cpu().numpy()
    out = {}
    for j in range(int(c[0])):
        p, st, n = (int(v) for v in g[j])
        out[p] = tuple(sorted(int(v) for v in l[st:st + n]))
    return out


def run(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))

    def emit(d):
        if rank == 0:
            print(json.dumps(d), flush=True)

    if world < 2:
        return emit({"verify_plans": "unavailable", "why": "the reference Buffer needs 2 or more ranks"})
    if not os.path.isdir(os.path.join(REF, "moonep")):
        return emit({"verify_plans": "unavailable", "why": "baseline/_ref/moonep is not installed on this machine"})
    dist.init_process_group("nccl")
    sys.path.insert(0, ROOT)
    from moonep_b200 import Buffer as Ours, routing
    S, H, K, epn, pad = 1024, 1024, 8, 16, 128
    E = epn * world
    cases = []
    for mv in SKEWS:
        scale = 0.0 if mv == 0 else routing.solve_scale_for_maxvio(mv, S, K, E, world, seed=3)[0]
        topk, w, tpe = (t.cuda() for t in routing.softmax_topk(S, K, E, scale, 3, rank))
        x = torch.randn(S, H, device="cuda", generator=torch.Generator(device="cuda").manual_seed(rank)).to(torch.bfloat16)
        cases.append((mv, topk.contiguous(), w.contiguous(), tpe.contiguous(), x))

    def collect(buf):
        res = []
        for mv, topk, w, tpe, x in cases:
            h, wn, cu, plan = buf.dispatch(x, w, topk, tpe)
            torch.cuda.synchronize()
            end = int(cu[-1])
            res.append(dict(dst=plan.dst.cpu(), cu=cu.cpu(), etc=plan.experts_to_copy.cpu(), zfr=plan.zero_fill_ranges.cpu(),
                            stats=plan.remote_stats.cpu(), dups=_dups(plan.dup_groups, plan.dup_loffs, plan.dup_counts),
                            rows=h[:end].cpu(), wts=wn[:end].cpu()))
        return res

    ours_buf = Ours(S, H, K, E, world, num_sms=16, token_padding=pad)
    ours = collect(ours_buf)
    ours_buf.check()
    ours_buf.destroy()
    dist.barrier()
    sys.path.insert(0, REF)
    from moonep import Buffer as Theirs
    ref_buf = Theirs(S=S, H=H, K=K, E=E, num_ep_ranks=world, num_sms=16, token_padding=pad)
    ref = collect(ref_buf)
    ref_buf.destroy()
    bad = []
    for (mv, *_), a, b in zip(cases, ours, ref):
        for key in ("dst", "cu", "etc", "zfr", "stats", "rows", "wts"):
            if not torch.equal(a[key], b[key]):
                bad.append(f"maxvio {mv}: {key}")
        if a["dups"] != b["dups"]:
            bad.append(f"maxvio {mv}: duplicate groups")
    flag = torch.tensor([len(bad)], device="cuda")
    dist.all_reduce(flag)
    emit({"verify_plans": "pass" if int(flag) == 0 else "fail", "n_gpus": world, "mismatches_all_ranks": int(flag),
          "rank0_mismatches": bad[:8], "config": {"S": S, "H": H, "K": K, "E": E, "token_padding": pad, "maxvio": list(SKEWS)},
          "compared": ["dst", "cu_seqlens", "experts_to_copy", "zero_fill_ranges", "remote_stats", "dup groups (sets)",
                       "dispatched rows", "dispatched route weights"]})
    dist.destroy_process_group()
