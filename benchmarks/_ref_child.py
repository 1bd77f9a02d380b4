"""Child process of the reference arm (see bench_reference.py)."""
import argparse
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
sys.path.insert(0, ROOT)

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--model", default="deepseek_v3")
    ap.add_argument("--maxvio", type=float, default=1.0)
    ap.add_argument("--no-sweep", action="store_true")
    args = ap.parse_args()
    from benchmarks import _ref_step
    _ref_step.run(args)
