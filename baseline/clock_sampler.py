"""SM clocks and throttle reasons sampled with nvidia-smi while a region is timed.

Shared by both arms of ``bench.py`` (this engine and the reference), so that the
two numbers carry clock records taken the same way.  Reading only: nothing here
changes a setting of the GPU.
"""

from __future__ import annotations

import subprocess
import threading
import time


class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples: list[list[str]] = []
        self.stamped: list[tuple[float, list[str]]] = []  # (arrival time, fields)
        self.proc = None
        self.t0 = self.t1 = None

    def mark_start(self):
        """The timed region starts now: samples from here on count (the tool needs a moment to
        come up, so it is started before the warm-up and the region is marked)."""
        self.t0 = time.time()

    def mark_end(self):
        self.t1 = time.time()

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "25"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.stamped.append((time.time(), parts))

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        lo = self.t0 if self.t0 is not None else 0.0
        hi = (self.t1 if self.t1 is not None else time.time()) + 0.03
        self.samples = [p for t, p in self.stamped if lo <= t <= hi] or [p for _, p in self.stamped[-1:]]
        mhz = sorted(int(s[0]) for s in self.samples if s[0].isdigit())
        mx = [int(s[1]) for s in self.samples if s[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i] == "Active" for s in self.samples)]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.samples)}
