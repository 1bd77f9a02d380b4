"""Multi-GPU tests: spawn one process per GPU (skipped with fewer than two devices)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.mark.parametrize("n", [2, 4, 8])
def test_dist_e2e(n):
    if _ngpu() < n:
        pytest.skip(f"needs {n} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", str(29500 + n), os.path.join(ROOT, "tests", "dist_e2e.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0, f"dist_e2e failed on {n} ranks:\n{r.stdout[-3000:]}\n{r.stderr[-3000:]}"
    assert "[dist_e2e] PASS" in r.stdout


@pytest.mark.parametrize("n", [2, 4, 8])
def test_dist_layer(n):
    """The fused MoE layer (push epilogue, ready flags, split launches) on real peers; see tests/dist_layer.py."""
    if _ngpu() < n:
        pytest.skip(f"needs {n} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", str(29520 + n), os.path.join(ROOT, "tests", "dist_layer.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env, cwd=ROOT)
    assert r.returncode == 0, f"dist_layer failed on {n} ranks:\n{r.stdout[-3000:]}\n{r.stderr[-3000:]}"
    assert "[dist_layer] PASS" in r.stdout


@pytest.mark.parametrize("n", [2, 4])
def test_rank_leaving_between_steps_is_detected_on_the_host(n):
    """Failure detection without a GPU fault: see tests/dist_peer_leave.py."""
    import json
    if _ngpu() < n:
        pytest.skip(f"needs {n} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", str(29540 + n), os.path.join(ROOT, "tests", "dist_peer_leave.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)
    assert r.returncode == 0, f"scenario failed on {n} ranks:\n{r.stdout[-3000:]}\n{r.stderr[-3000:]}"
    res = {}
    for line in r.stdout.splitlines():
        if line.startswith("RESULT "):
            d = json.loads(line[len("RESULT "):])
            res[d["rank"]] = d
    assert sorted(res) == list(range(n)), r.stdout[-2000:]
    for rank, d in res.items():
        assert d["steps"] == 3 and d["wrong"] == 0, d
        assert d["status"] == ("left" if rank == n - 1 else f"lost:{n - 1}@3"), d
