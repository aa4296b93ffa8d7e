"""Sampling of SM clocks, power and throttle reasons while a benchmark's timed
region runs.  Read-only: nothing here changes a GPU setting.  NVML is polled
from a background thread (a few milliseconds per sample); ``nvidia-smi`` is the
fallback when the NVML bindings are missing."""
from __future__ import annotations

import os
import shutil
import signal
import statistics
import subprocess
import tempfile
import threading
import time
from typing import Optional

_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
          "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
          "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


def _physical_index(cuda_index: int) -> int:
    """nvidia-smi / NVML index of a CUDA device index under CUDA_VISIBLE_DEVICES."""
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        ids = [v.strip() for v in vis.split(",") if v.strip()]
        if cuda_index < len(ids) and ids[cuda_index].isdigit():
            return int(ids[cuda_index])
    return cuda_index


class ClockSampler:
    """``with ClockSampler(cuda_index) as s: ...`` then ``s.summary()``."""

    def __init__(self, gpu_index: int = 0, period_ms: float = 5.0):
        self.gpu_index = _physical_index(gpu_index)
        self.period_ms = period_ms
        self._samples: list[tuple[float, float, float, int]] = []  # (sm, max_sm, power_w, reasons)
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._proc: Optional[subprocess.Popen] = None
        self._path: Optional[str] = None
        self._nvml = None
        self._handle = None
        self._max_sm = 0.0

    # ---- NVML thread -----------------------------------------------------
    def _sample(self):
        nv, h = self._nvml, self._handle
        try:
            sm = float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
            power = nv.nvmlDeviceGetPowerUsage(h) / 1000.0
            reasons = int(nv.nvmlDeviceGetCurrentClocksEventReasons(h))
            self._samples.append((sm, self._max_sm, power, reasons))
        except Exception:
            pass

    def _run(self):
        while not self._stop.is_set():
            self._sample()
            time.sleep(self.period_ms / 1000.0)

    def __enter__(self):
        try:
            import pynvml

            # library and device handle are set up before the sampled region starts: a short region
            # (a few tens of milliseconds) would otherwise be over before the first sample
            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(self.gpu_index)
            self._max_sm = float(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
            return self
        except Exception:
            self._nvml = None
        if shutil.which("nvidia-smi") is None:
            return self
        fd, self._path = tempfile.mkstemp(prefix="fo_clocks_", suffix=".csv")
        os.close(fd)
        out = open(self._path, "w")
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={_QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=out, stderr=subprocess.DEVNULL)
        except OSError:
            self._proc = None
        finally:
            out.close()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
            self._sample()  # one more right at the end of the region: the GPU has not yet clocked down
        if self._proc is not None:
            self._proc.send_signal(signal.SIGINT)
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()
        return False

    def _from_csv(self):
        names = [(0x8, "hw_slowdown"), (0x40, "hw_thermal_slowdown"), (0x20, "sw_thermal_slowdown"),
                 (0x4, "sw_power_cap")]
        if not self._path or not os.path.exists(self._path):
            return
        with open(self._path) as f:
            for line in f:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm, mx, power = float(parts[1]), float(parts[2]), float(parts[3])
                except ValueError:
                    continue
                bits = 0
                for (bit, _), val in zip(names, parts[5:9]):
                    if val.lower().startswith("active"):
                        bits |= bit
                self._samples.append((sm, mx, power, bits))
        try:
            os.unlink(self._path)
        except OSError:
            pass

    def summary(self) -> dict:
        """Median SM clock over the samples taken under load (power at least
        60 % of the highest power seen), and every throttle reason seen there."""
        if self._nvml is None:
            self._from_csv()
        res = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": len(self._samples),
               "samples_under_load": 0, "power_w_max": None}
        if not self._samples:
            return res
        pmax = max(s[2] for s in self._samples)
        busy = [s for s in self._samples if s[2] >= 0.6 * pmax] or self._samples
        bits = 0
        for s in busy:
            bits |= s[3]
        # NVML clocks-event-reason bits
        names = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
                 0x80: "hw_power_brake_slowdown"}
        res.update(sm_mhz=statistics.median(s[0] for s in busy), sm_max_mhz=max(s[1] for s in self._samples),
                   samples_under_load=len(busy), power_w_max=round(pmax, 1),
                   reasons=sorted(n for b, n in names.items() if bits & b))
        return res
