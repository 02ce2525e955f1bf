"""Read-only sampling of SM clocks and throttle reasons with ``nvidia-smi`` while a timed region runs, so that every
number a benchmark script prints carries the clocks it was measured under (time x median MHz allows comparing runs
taken at different clocks). Nothing here changes a GPU setting."""
from __future__ import annotations

import subprocess
import threading

QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler(threading.Thread):
    def __init__(self, gpu_index: int = 0, period_ms: int = 100):
        super().__init__(daemon=True)
        self.gpu, self.period = gpu_index, period_ms
        self.samples: list = []
        self.proc = None

    def run(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={QUERY}", "--format=csv,noheader,nounits", "-lms", str(self.period),
                                          "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            for line in self.proc.stdout:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) >= 9:
                    self.samples.append(parts)
        except Exception:  # noqa: BLE001 - a missing nvidia-smi leaves the record empty
            pass

    def stop(self) -> dict:
        if self.proc is not None:
            self.proc.terminate()
        rows = list(self.samples)
        sm = sorted(float(s[1]) for s in rows if s[1].replace(".", "").isdigit())
        mx = [float(s[2]) for s in rows if s[2].replace(".", "").isdigit()]
        reasons = set()
        for s in rows:
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(rows)}
