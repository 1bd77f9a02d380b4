"""Throughput of the tcgen05 grouped GEMM modes at an MoE shape, device-timed, against the
measured cuBLAS bf16 peak (MEASURED_PEAKS.json when present).

    python benchmarks/bench_gemm.py [--rows 32768 --H 7168 --Hp 2048 --groups 32]
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from moonep_b200.ops import grouped_gemm as gg  # noqa: E402


def timed(fn, warmup=3, iters=10):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=32768)
    ap.add_argument("--H", type=int, default=7168)
    ap.add_argument("--Hp", type=int, default=2048)
    ap.add_argument("--groups", type=int, default=32)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--only", default="", help="comma-separated subset of modes")
    a = ap.parse_args()
    G, H, Hp, rows = a.groups, a.H, a.Hp, a.rows
    per = rows // G // 128 * 128
    cu = torch.tensor([per * (i + 1) for i in range(G)], dtype=torch.int32, device="cuda")
    rows = per * G
    bf = dict(dtype=torch.bfloat16, device="cuda")
    x = torch.randn(rows, H, **bf)
    wg = torch.randn(G, H, Hp, **bf) * 0.02
    wu = torch.randn(G, H, Hp, **bf) * 0.02
    wd = torch.randn(G, Hp, H, **bf) * 0.02
    act = torch.empty(rows, Hp, **bf)
    gu = torch.empty(rows, 2 * Hp, **bf)
    y = torch.empty(rows, H, **bf)
    dA = torch.empty(rows, Hp, **bf)
    dWg = torch.empty(G, H, Hp, device="cuda")
    dWd = torch.empty(G, Hp, H, device="cuda")
    upd_all = torch.ones(G, dtype=torch.int32, device="cuda")
    peak = None
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        peak = json.load(open(p)).get("bf16_tflops")
    cases = {
        "gate_up": (lambda: gg.gate_up(x, wg, wu, cu, act, gu), 2 * 2 * rows * H * Hp),
        "down": (lambda: gg.down(act, wd, cu, y), 2 * rows * H * Hp),
        "dgrad_down": (lambda: gg.dgrad(y, wd, cu, dA), 2 * rows * H * Hp),
        "dgrad_gate_up": (lambda: gg.dgrad_gate_up(gu, wg, wu, cu, y), 2 * 2 * rows * H * Hp),
        "wgrad_gate": (lambda: gg.wgrad(x, gu[:, :Hp], cu, dWg), 2 * rows * H * Hp),
        "wgrad_down": (lambda: gg.wgrad(act, y, cu, dWd), 2 * rows * H * Hp),
        # optimizer in the epilogue: every group's bf16 weights are updated, no fp32 gradient is written
        "wgrad_gate_sgd_epilogue": (lambda: gg.wgrad(x, gu[:, :Hp], cu, dWg, update=(wg, 1e-6, upd_all)), 2 * rows * H * Hp),
        "sgd_step_gate": (lambda: gg.sgd_step(wg, dWg, 1e-6), 0),
    }
    only = [m for m in a.only.split(",") if m]
    for name, (fn, flops) in cases.items():
        if only and name not in only:
            continue
        ms = timed(fn, warmup=a.warmup, iters=a.iters)
        tf = flops / ms / 1e9
        row = {"mode": name, "ms": round(ms, 4), "tflops": round(tf, 1)}
        if not flops:          # a memory-bound helper: report bytes instead (fp32 gradient + bf16 weights read, weights written)
            row = {"mode": name, "ms": round(ms, 4), "GBps": round(G * H * Hp * 8 / ms / 1e6, 1)}
            print(json.dumps(row))
            continue
        if peak:
            row["frac_of_measured_cublas_peak"] = round(tf / peak, 3)
        print(json.dumps(row))
    if only:
        gg.check_status()
        return
    t = torch.matmul  # cuBLAS reference point at a comparable dense shape
    a_ = torch.randn(rows, H, **bf); b_ = torch.randn(H, Hp, **bf)
    ms = timed(lambda: t(a_, b_), iters=a.iters)
    print(json.dumps({"mode": "cublas_dense_same_flops_as_down", "ms": round(ms, 4), "tflops": round(2 * rows * H * Hp / ms / 1e9, 1)}))
    gg.check_status()


if __name__ == "__main__":
    main()
