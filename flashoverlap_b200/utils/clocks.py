"""Sampling of SM clocks and throttle reasons with ``nvidia-smi`` while a
benchmark's timed region runs.  Read-only: nothing here changes a GPU setting."""
from __future__ import annotations

import os
import shutil
import signal
import statistics
import subprocess
import tempfile
from typing import Optional

_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
          "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
          "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    """``with ClockSampler(gpu_index) as s: ...`` then ``s.summary()``."""

    def __init__(self, gpu_index: int = 0, period_ms: int = 100):
        self.gpu_index = gpu_index
        self.period_ms = period_ms
        self._proc: Optional[subprocess.Popen] = None
        self._path: Optional[str] = None

    def __enter__(self):
        if shutil.which("nvidia-smi") is None:
            return self
        fd, self._path = tempfile.mkstemp(prefix="fo_clocks_", suffix=".csv")
        os.close(fd)
        out = open(self._path, "w")
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={_QUERY}", "--format=csv,noheader,nounits",
                 "-lms", str(self.period_ms)],
                stdout=out, stderr=subprocess.DEVNULL)
        except OSError:
            self._proc = None
        finally:
            out.close()
        return self

    def __exit__(self, *exc):
        if self._proc is not None:
            self._proc.send_signal(signal.SIGINT)
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()
        return False

    def summary(self) -> dict:
        res = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "power_w_max": None}
        if not self._path or not os.path.exists(self._path):
            return res
        sm, mx, power = [], [], []
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self._path) as f:
            for line in f:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1]))
                    mx.append(float(parts[2]))
                    power.append(float(parts[3]))
                except ValueError:
                    continue
                for name, val in zip(names, parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        try:
            os.unlink(self._path)
        except OSError:
            pass
        if sm:
            # under load = the upper half of the samples (idle gaps between steps pull clocks down)
            busy = sorted(sm)[len(sm) // 2:]
            res.update(sm_mhz=statistics.median(busy), sm_max_mhz=max(mx), samples=len(sm),
                       power_w_max=max(power), reasons=sorted(reasons))
        return res
