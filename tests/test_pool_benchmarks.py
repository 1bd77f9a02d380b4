"""The prefetch / reduce_grad benchmarks: their slot-table builder on CPU, and a small
emulated-rank run of each script on a GPU."""
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "benchmarks"))

import _pool_bench as pb  # noqa: E402


@pytest.mark.parametrize("R", [2, 3, 4, 8])
def test_slot_table_builder(R):
    for owner in (0, R - 1):
        for case in pb.cases_for(R, 256, 128):
            epn = case["epn"]
            etc = pb.experts_to_copy_for(R, epn, owner, case["counts"])
            assert etc.shape == (R, epn) and etc.dtype == torch.int32
            assert int((etc >= 0).sum()) == sum(case["counts"])
            assert (etc[owner] == -1).all(), "an owner never holds a copy of its own expert"
            for d in range(R):
                live = etc[d][etc[d] >= 0]
                assert (etc[d, live.numel():] == -1).all(), "live slots come first"
                assert (live[1:] > live[:-1]).all(), "slots list experts in ascending order, no repeats"
                assert ((live // epn) == owner).all()
            # every expert sits on as many distinct ranks as its fan-out asks for
            for e, cnt in enumerate(case["counts"]):
                assert int((etc == owner * epn + e).any(dim=1).sum()) == cnt


def test_synthetic_plan_shapes():
    etc = pb.experts_to_copy_for(4, 4, 1, [3, 1, 0, 2])
    plan = pb.synthetic_plan(etc, NvS=256, K=2, N=16, device="cpu")
    assert plan.R == 4 and plan.E == 16 and torch.equal(plan.experts_to_copy, etc)


@pytest.mark.gpu
@pytest.mark.parametrize("script,rate", [("bench_prefetch.py", "owner_egress_GBps"),
                                          ("bench_grad_reduce.py", "owner_ingress_GBps")])
def test_pool_benchmark_scripts_run_emulated(script, rate, cuda_device):
    cmd = [sys.executable, os.path.join(ROOT, "benchmarks", script), "--emulate-ranks", "4", "--H", "256",
           "--Hp", "128", "--num-sms", "4", "--iters", "3", "--warmup", "1", "--cases", "slots_3", "ramp", "epn4_full"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    rows = [json.loads(line) for line in out.stdout.splitlines() if line.startswith("{")]
    assert [r["case"] for r in rows] == ["slots_3", "ramp", "epn4_full"]
    for r in rows:
        assert r["slots"] > 0 and r["us"] > 0 and r[rate] > 0 and r["emulated"] is True


@pytest.mark.gpu
@pytest.mark.parametrize("mode", [[], ["--no-cudagraph"]], ids=["cudagraph", "eager"])
def test_comm_benchmark_script_runs(mode, cuda_device, tmp_path):
    out_csv = tmp_path / "comm.csv"
    cmd = [sys.executable, os.path.join(ROOT, "benchmarks", "bench_comm.py"), "--S", "256", "--hidden", "256", "512",
           "--topk", "4", "--epn", "4", "--maxvio", "0", "1", "--num-sms", "4", "--pad", "16", "--iters", "3",
           "--warmup", "1", "--out", str(out_csv), *mode]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    rows = [json.loads(line) for line in out.stdout.splitlines() if line.startswith("{")]
    assert len(rows) == 4 and {r["H"] for r in rows} == {256, 512}
    for r in rows:
        assert all(r[k + "_us"] > 0 for k in ("dispatch_fwd", "dispatch_bwd", "combine_fwd", "combine_bwd"))
        assert r["timing"] == ("eager" if mode else "cudagraph")
    assert out_csv.read_text().count("\n") == 5
