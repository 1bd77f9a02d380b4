"""Host-only checks of argument validation (no GPU): num_sms is validated before any CUDA
or process-group access, like the reference (tests/test_api_validation.py:8-86)."""
import os

import pytest

from moonep_b200.api import validate_num_sms, num_sms_dedup_from_env
from moonep_b200.geometry import Geometry


def _boom():
    raise AssertionError("device must not be queried for an invalid num_sms")


@pytest.mark.parametrize("bad", [True, 1.5, "8", [4]])
def test_num_sms_type(bad):
    with pytest.raises(TypeError, match="num_sms must be a positive int"):
        validate_num_sms(bad, _boom)


@pytest.mark.parametrize("bad", [0, -3])
def test_num_sms_range(bad):
    with pytest.raises(ValueError, match="num_sms must be a positive int"):
        validate_num_sms(bad, _boom)


def test_num_sms_vs_device():
    assert validate_num_sms(None, lambda: 148) == (32, 148)
    assert validate_num_sms(None, lambda: 16) == (16, 16)
    assert validate_num_sms(20, lambda: 148) == (20, 148)
    with pytest.raises(ValueError, match="must not exceed the device SM count"):
        validate_num_sms(200, lambda: 148)


def test_buffer_rejects_bad_num_sms_before_cuda(monkeypatch):
    import torch
    from moonep_b200.api import Buffer
    monkeypatch.setattr(torch.cuda, "current_device", _boom)
    with pytest.raises(TypeError):
        Buffer(8, 64, 2, 4, 1, num_sms="x")
    with pytest.raises(ValueError):
        Buffer(8, 64, 2, 4, 1, num_sms=0)


def test_dedup_env(monkeypatch):
    monkeypatch.delenv("MOONEP_NUM_SMS_DEDUP", raising=False)
    assert num_sms_dedup_from_env(148) == 148
    monkeypatch.setenv("MOONEP_NUM_SMS_DEDUP", "12")
    assert num_sms_dedup_from_env(148) == 12
    monkeypatch.setenv("MOONEP_NUM_SMS_DEDUP", "abc")
    with pytest.raises(ValueError):
        num_sms_dedup_from_env(148)
    monkeypatch.setenv("MOONEP_NUM_SMS_DEDUP", "0")
    with pytest.raises(ValueError):
        num_sms_dedup_from_env(148)


def test_geometry_limits():
    g = Geometry.make(4096, 7168, 8, 256, 8, 128, 32)
    assert g.NvS == 40960 and g.epn == 32 and g.N == 32768
    with pytest.raises(AssertionError, match="divisible"):
        Geometry.make(8, 64, 2, 5, 2)
    with pytest.raises(AssertionError, match="K <= 32"):
        Geometry.make(8, 64, 33, 64, 2)
    with pytest.raises(AssertionError, match="R <= 128"):
        Geometry.make(8, 64, 2, 256, 256)
    with pytest.raises(AssertionError, match="multiple of 8"):
        Geometry.make(8, 60, 2, 4, 2)
    with pytest.raises(AssertionError, match="token_padding"):
        Geometry.make(8, 64, 2, 4, 2, token_padding=0)


def test_geometry_push_combine_regions():
    """The push-combine regions are only laid out on request, follow the regular regions and do
    not overlap: provenance table [NvS] int32, receive area [S*K, H] bf16, scalars [S*K] fp32."""
    a = Geometry.make(4096, 7168, 8, 256, 8, 128, 32)
    b = Geometry.make(4096, 7168, 8, 256, 8, 128, 32, push_combine=True)
    assert (a.off_srcinfo, a.off_push, a.off_pushw) == (0, 0, 0)
    assert b.off_srcinfo >= a.chunk_bytes - 1024 and b.off_srcinfo % 1024 == 0
    assert b.off_push >= b.off_srcinfo + b.NvS * 4 and b.off_push % 1024 == 0
    assert b.off_pushw >= b.off_push + b.N * b.H * 2
    assert b.chunk_bytes >= b.off_pushw + b.N * 4
    for name in ("off_hidden", "off_weights", "off_tpe", "off_bar", "off_dupcnt", "off_dupgroups", "off_duploffs", "off_ready"):
        assert getattr(a, name) == getattr(b, name)


def test_pool_layout_and_description():
    """Offsets of the [local | slots] pools: disjoint, 1 KiB aligned, weights before grads; the
    text diagram names every projection and view."""
    import torch
    from moonep_b200.pools import pool_layout, describe_layout, NAMES
    shapes = {"gate": (256, 96), "up": (256, 96), "down": (96, 256)}
    epn = 3
    woff, goff, total = pool_layout(epn, shapes, torch.bfloat16, True)
    spans = []
    for n in NAMES:
        r, c = shapes[n]
        spans.append((woff[n], woff[n] + 2 * epn * r * c * 2))
        spans.append((goff[n], goff[n] + 2 * epn * r * c * 4))
    spans.sort()
    assert all(a % 1024 == 0 for a, _ in spans)
    assert all(spans[i][1] <= spans[i + 1][0] for i in range(len(spans) - 1)) and spans[-1][1] <= total
    assert max(woff.values()) < min(goff.values())
    assert pool_layout(epn, shapes, torch.int8, False)[1] == {}
    text = describe_layout(epn, shapes, torch.bfloat16, True, world=4)
    for word in ("gate", "up", "down", "prefetch", "reduce", "compute", "[R=4, epn=3"):
        assert word in text


def test_bench_keeps_stdout_for_the_result_line():
    """bench.py prints exactly one line on stdout even if a library writes banners there."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = ("import os, sys; sys.path.insert(0, %r); import bench; bench._reserve_stdout(); "
            "print('banner from python'); os.write(1, b'banner from C\\n'); bench._emit('{\"ok\": 1}')" % root)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr
    assert r.stdout == '{"ok": 1}\n'
    assert "banner from python" in r.stderr and "banner from C" in r.stderr


def test_grad_reduce_ring_geometry():
    """Index arithmetic of grad_reduce's per-warp stage, restated on the host: with up to eight
    replicas a unit takes ns*P of the 32 slots and the ring holds four units that never overlap;
    beyond that one unit uses the stage alone (constants mirror csrc/device/grad_reduce.cu)."""
    SLOTS, DEPTH = 32, 4
    for ns in range(1, 200):
        ring = ns * DEPTH <= SLOTS
        P = max(1, min(8, SLOTS // (ns * DEPTH if ring else ns)))
        if ring:
            spans = [(r * ns * P, (r + 1) * ns * P) for r in range(DEPTH)]
            assert spans[-1][1] <= SLOTS
            assert all(spans[i][1] <= spans[i + 1][0] for i in range(DEPTH - 1))
            # slot of (unit r, replica j, vector p) is unique
            idx = {(r * ns * P + j * P + p) for r in range(DEPTH) for j in range(ns) for p in range(P)}
            assert len(idx) == DEPTH * ns * P
        else:
            per_pass = min(ns, SLOTS)
            assert per_pass * P <= SLOTS
    assert [max(1, min(8, SLOTS // (ns * DEPTH))) for ns in (1, 2, 3, 4, 8)] == [8, 4, 2, 2, 1]


def test_clock_sampler_with_a_fake_nvidia_smi(tmp_path, monkeypatch):
    """The sampler reads clocks and throttle reasons from nvidia-smi's CSV stream; "under load"
    is decided by power draw, because a power-capped GPU clocks down when it is busy."""
    import stat
    import time
    from moonep_b200.utils.clocks import ClockSampler, under_load
    fake = tmp_path / "nvidia-smi"
    fake.write_text(
        "#!/bin/bash\n"
        "echo '0, 1965, 1965, 180.5, 0x0000000000000000, Not Active, Not Active, Not Active, Not Active'\n"
        "for i in 1 2 3 4 5 6; do\n"
        "  echo '0, 1410, 1965, 995.0, 0x0000000000000004, Not Active, Not Active, Not Active, Active'\n"
        "done\n"
        "echo '0, 1965, 1965, 210.0, 0x0000000000000000, Not Active, Not Active, Not Active, Not Active'\n"
        "sleep 30\n")
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", f"{tmp_path}:{os.environ['PATH']}")
    s = ClockSampler(0, 20).start()
    time.sleep(0.3)
    out = s.stop()
    assert out["samples"] == 8 and out["sm_max_mhz"] == 1965.0
    assert out["sm_mhz"] == 1410.0, "the busy samples are the power-capped ones, not the idle 1965 MHz ones"
    assert out["reasons"] == ["sw_power_cap"]
    # no usable power reading: fall back to the upper half of the clock samples
    assert under_load([300.0, 300.0, 1900.0, 1950.0], [None] * 4) == [1900.0, 1950.0]
    assert under_load([1965.0, 1400.0, 1420.0], [100.0, 990.0, 1000.0]) == [1400.0, 1420.0]
