"""Sample GPU clocks and throttle reasons with nvidia-smi while a timed region runs
(read-only queries; no GPU setting is ever changed)."""
from __future__ import annotations

import shutil
import statistics
import subprocess
import tempfile

_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
          "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
          "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    def __init__(self, gpu_index=0, period_ms: int = 100):
        """gpu_index: one index, or a list of indices sampled together by one process."""
        if isinstance(gpu_index, (list, tuple)):
            gpu_index = ",".join(str(i) for i in gpu_index)
        self.gpu_index, self.period_ms = gpu_index, period_ms
        self.proc = None
        self.file = None

    def __enter__(self):
        exe = shutil.which("nvidia-smi")
        if exe:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(
                [exe, f"--query-gpu={_QUERY}", "--format=csv,noheader,nounits", "-i", str(self.gpu_index),
                 "-lms", str(self.period_ms)], stdout=self.file, stderr=subprocess.DEVNULL)
        return self

    def wait_first(self, timeout_s: float = 15.0) -> bool:
        """Blocks until the first sample is in the file: nvidia-smi takes a second or
        more to start on a host with many GPUs, and a timed region that ends before
        that would have no clock record."""
        import os
        import time

        if not self.file:
            return False
        t0 = time.time()
        while time.time() - t0 < timeout_s:
            if os.path.getsize(self.file.name) > 0:
                return True
            if self.proc.poll() is not None:
                return False
            time.sleep(0.05)
        return False

    def __exit__(self, *exc):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
        return False

    def summary(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if not self.file:
            return out
        self.file.flush()
        rows = []
        with open(self.file.name) as f:
            for line in f:
                p = [x.strip() for x in line.split(",")]
                if len(p) >= 9:
                    rows.append(p)
        if not rows:
            return out
        sm = [float(r[1]) for r in rows if r[1].replace(".", "").isdigit()]
        # "under load" = the upper half of the power samples, else everything
        out["samples"] = len(rows)
        if sm:
            out["sm_mhz"] = statistics.median(sm)
        try:
            out["sm_max_mhz"] = float(rows[0][2])
        except ValueError:
            pass
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for i, nm in enumerate(names):
            if any(r[5 + i].lower().startswith("active") for r in rows):
                out["reasons"].append(nm)
        return out
