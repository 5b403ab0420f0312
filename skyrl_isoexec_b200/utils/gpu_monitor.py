"""Read-only GPU monitor (reference: the Ray GPU utilisation monitor of R/train/utils/ray_gpu_monitor.py, and the clock
record every benchmark number here carries). A daemon thread polls ``nvidia-smi --query-gpu`` for one GPU: SM clock,
maximum SM clock, power draw, utilisation, memory used and the clock-event reasons. Nothing is ever set."""

from __future__ import annotations

import subprocess
import threading
import time

QUERY = ("clocks.sm,clocks.max.sm,power.draw,utilization.gpu,memory.used,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
REASONS = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")


def parse_row(line: str) -> dict | None:
    """One CSV line of the query above -> numbers and the set of active reasons (None if it does not parse)."""
    parts = [x.strip() for x in line.split(",")]
    if len(parts) < 5:
        return None
    try:
        nums = [float(x) for x in parts[:5]]
    except ValueError:
        return None
    active = {name for name, v in zip(REASONS, parts[5:9]) if v.lower().startswith("active")}
    return {"sm_mhz": nums[0], "sm_max_mhz": nums[1], "power_w": nums[2], "util_pct": nums[3], "mem_mib": nums[4], "reasons": active}


class GpuMonitor(threading.Thread):
    def __init__(self, index: int, period_s: float = 0.2, runner=None):
        super().__init__(daemon=True)
        self.index, self.period_s, self.rows, self.stop_flag = index, period_s, [], False
        self._run_query = runner or self._nvidia_smi

    def _nvidia_smi(self) -> str:
        return subprocess.run(["nvidia-smi", f"--query-gpu={QUERY}", "--format=csv,noheader,nounits", "-i", str(self.index)],
                              capture_output=True, text=True, timeout=5).stdout.strip()

    def run(self):
        while not self.stop_flag:
            try:
                row = parse_row(self._run_query())
                if row:
                    self.rows.append(row)
            except Exception:  # noqa: BLE001 - monitoring never takes the job down
                pass
            time.sleep(self.period_s)

    def stop(self) -> dict:
        self.stop_flag = True
        if self.is_alive():
            self.join(timeout=2)
        return self.summary()

    def summary(self, reset: bool = False) -> dict:
        rows = list(self.rows)
        if reset:
            self.rows.clear()
        if not rows:
            return {"sm_mhz": 0, "sm_max_mhz": 0, "reasons": [], "samples": 0}
        med = lambda k: sorted(r[k] for r in rows)[len(rows) // 2]
        reasons = sorted(set().union(*(r["reasons"] for r in rows)))
        return {"sm_mhz": int(med("sm_mhz")), "sm_max_mhz": int(max(r["sm_max_mhz"] for r in rows)), "power_w": round(med("power_w"), 1),
                "util_pct": round(med("util_pct"), 1), "mem_mib": int(max(r["mem_mib"] for r in rows)), "reasons": reasons,
                "samples": len(rows)}
