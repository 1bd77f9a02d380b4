"""Reference arm of bench.py: the UNMODIFIED reference package (installed under
``baseline/_ref``) drives dispatch / prefetch / combine / reduce_grad through its own public
``moonep.Buffer`` API; the expert FFN, which the reference does not ship, is plain PyTorch
(library GEMMs per expert group).  Nothing from ``moonep_b200`` is imported on this path.

The step runs in a child process per rank: the reference reports driver errors by calling
``exit()`` (csrc/nvl_shared_buffer.cuh:17-39 of the reference), which must not take the
benchmark driver down; a child that dies without a result becomes an ``unavailable`` line.
"""

import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")


def unavailable(why: str):
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": " ".join(why.split())[:400]}), flush=True)


def run_reference(args):
    if not os.path.isdir(os.path.join(REF, "moonep")):
        return unavailable("baseline/_ref/moonep is not installed on this machine")
    try:
        import torch
        if not torch.cuda.is_available():
            return unavailable("no CUDA device")
    except Exception as exc:
        return unavailable(f"torch import failed: {exc}")
    cmd = [sys.executable, os.path.join(ROOT, "benchmarks", "_ref_child.py"), "--steps", str(args.steps),
           "--warmup", str(args.warmup), "--model", args.model, "--maxvio", str(args.maxvio)]
    if args.no_sweep:
        cmd.append("--no-sweep")
    try:
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=1500, cwd=ROOT)
    except subprocess.TimeoutExpired:
        return unavailable("the reference step did not finish within 1500 s")
    line = next((l for l in reversed(r.stdout.splitlines()) if l.startswith("{") and '"metric"' in l), None)
    if line is not None:
        print(line, flush=True)
        return
    if int(os.environ.get("RANK", "0")) != 0 and r.returncode == 0:
        return
    tail = [l for l in (r.stdout + "\n" + r.stderr).splitlines() if l.strip() and "Warning" not in l and "warn" not in l]
    unavailable(f"reference step exited with code {r.returncode}: {tail[-1] if tail else 'no output'}")
