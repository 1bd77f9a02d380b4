"""A few training steps of one MoE block on one GPU, launched from Python, for a per-kernel
launch list:

    ncu --metrics gpu__time_duration.sum --clock-control none --csv --log-file launches.csv \
        python benchmarks/profile_step.py --model deepseek_v3 --steps 3

(one pass per kernel; the last step's rows are the ones to read).  Without a profiler it just
prints the device-timed step.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from moonep_b200.models.moe_block import CONFIGS, MoEBlock  # noqa: E402
from moonep_b200.ops import grouped_gemm as gg  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="deepseek_v3", choices=sorted(CONFIGS))
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--skew", type=float, default=0.35, help="scale of the router bias (0 = balanced routing)")
    a = ap.parse_args()
    cfg = CONFIGS[a.model]
    blk = MoEBlock(cfg, num_sms=32, seed=0, router_skew=a.skew)
    x = torch.randn(cfg.S, cfg.H, device="cuda").to(torch.bfloat16)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i in range(a.steps):
        if i == a.steps - 1:
            torch.cuda.synchronize()
            e0.record()
        xi = x.detach().requires_grad_(True)
        loss = (blk.forward(xi).float() ** 2).mean()
        loss.backward()
        blk.sgd_step(1e-3)
    e1.record()
    torch.cuda.synchronize()
    blk.buf.check()
    gg.check_status()
    print(f"{a.model}: last step {e0.elapsed_time(e1):.3f} ms, loss {float(loss):.5f}")
    blk.destroy()


if __name__ == "__main__":
    main()
