"""Sample GPU clocks and throttle reasons with nvidia-smi while a timed region runs
(read-only: nothing about the GPU is changed)."""

from __future__ import annotations

import os
import shutil
import statistics
import subprocess
import tempfile

QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    def __init__(self, device_index: int = 0, period_ms: int = 20):
        self.device_index, self.period_ms = device_index, period_ms
        self._proc, self._path = None, None

    def start(self):
        exe = shutil.which("nvidia-smi")
        if exe is None:
            return self
        fd, self._path = tempfile.mkstemp(prefix="mep_clocks_", suffix=".csv")
        os.close(fd)
        self._proc = subprocess.Popen([exe, f"--query-gpu={QUERY}", "--format=csv,noheader,nounits",
                                       "-i", str(self.device_index), "-lms", str(self.period_ms)],
                                      stdout=open(self._path, "w"), stderr=subprocess.DEVNULL)
        # nvidia-smi can take seconds to come up on a multi-GPU box: wait for its first sample
        import time
        t0 = time.time()
        while time.time() - t0 < 20.0 and os.path.getsize(self._path) == 0 and self._proc.poll() is None:
            time.sleep(0.05)
        return self

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self._proc is None:
            return out
        self._proc.terminate()
        try:
            self._proc.wait(timeout=5)
        except Exception:
            self._proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        try:
            for line in open(self._path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1])); mx.append(float(f[2]))
                except ValueError:
                    continue
                try:
                    pw.append(float(f[3]))
                except ValueError:
                    pw.append(None)
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
        finally:
            try:
                os.unlink(self._path)
            except OSError:
                pass
        if sm:
            out.update(sm_mhz=statistics.median(under_load(sm, pw)), sm_max_mhz=max(mx), reasons=sorted(reasons),
                       samples=len(sm))
        return out


def under_load(sm, power):
    """SM clock samples taken while the GPU was busy.  Busy = power draw of at least 60 % of the
    highest draw seen (a power-capped GPU clocks DOWN under load, so the clock itself cannot tell
    busy from idle); without usable power readings, the upper half of the clock samples."""
    known = [p for p in power if p is not None]
    if len(known) == len(sm) and known and max(known) > 0:
        cut = 0.6 * max(known)
        hot = [c for c, p in zip(sm, power) if p >= cut]
        if hot:
            return hot
    return sorted(sm)[len(sm) // 2:]
