"""Reference arm of bench.py: the UNMODIFIED reference package (installed under
``baseline/_ref``) drives dispatch / prefetch / combine / reduce_grad through its own public
``moonep.Buffer`` API; the expert FFN, which the reference does not ship, is plain PyTorch
(library GEMMs per expert group).  Nothing from ``moonep_b200`` is imported on this path.
"""

import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")


def unavailable(why: str):
    print(json.dumps({"impl": "reference", "unavailable": why.replace("\n", " ")[:400]}), flush=True)


def run_reference(args):
    if not os.path.isdir(os.path.join(REF, "moonep")):
        return unavailable("baseline/_ref/moonep is not installed on this machine")
    sys.path.insert(0, REF)
    try:
        import torch
        if not torch.cuda.is_available():
            return unavailable("no CUDA device")
        from benchmarks import _ref_step
        return _ref_step.run(args)
    except Exception as exc:  # the reference could not be imported / JIT-built / run
        return unavailable(f"{type(exc).__name__}: {exc}")
