"""GPU clock sampling during a timed region (reads only; nothing is ever set)."""
from __future__ import annotations

import statistics
import subprocess
import threading
from typing import Dict, List, Optional

_FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
           "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
           "clocks_event_reasons.sw_power_cap")


class ClockSampler:
    """``with ClockSampler(index) as c: ...`` then ``c.summary()``."""

    def __init__(self, gpu_index: int = 0, period_ms: int = 200):
        self.gpu, self.period = gpu_index, period_ms
        self.lines: List[str] = []
        self._proc: Optional[subprocess.Popen] = None
        self._thr: Optional[threading.Thread] = None

    def __enter__(self):
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={_FIELDS}", "--format=csv,noheader,nounits", "-lms", str(self.period)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self._thr = threading.Thread(target=self._pump, daemon=True)
            self._thr.start()
        except OSError:
            self._proc = None
        return self

    def _pump(self):
        assert self._proc and self._proc.stdout
        for line in self._proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self._proc:
            self._proc.terminate()          # the exact child started above
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()
        return False

    def summary(self) -> Dict:
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}
