"""Timing hygiene helpers shared by bench.py and the per-workload benchmarks.

* ``ClockSampler`` samples ``nvidia-smi`` clocks and throttle reasons in a background process while a timed region runs
  and summarises them (median SM MHz under load, max SM MHz, active reasons).
* ``device_time_ms`` times a callable with CUDA events on the current stream after a synchronize on both sides.
* ``flush_l2`` overwrites a buffer larger than L2 between timed iterations.
"""
from __future__ import annotations

import os
import shutil
import statistics
import subprocess
import tempfile
from typing import Callable, Dict, List, Optional

_QUERY = (
    "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
    "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
    "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
)


class ClockSampler:
    """Context manager: ``with ClockSampler(gpu_index) as cs: ...; cs.summary()``."""

    def __init__(self, gpu_index: int = 0, period_ms: int = 100):
        self.gpu_index = gpu_index
        self.period_ms = period_ms
        self._proc: Optional[subprocess.Popen] = None
        self._path: Optional[str] = None

    def __enter__(self) -> "ClockSampler":
        exe = shutil.which("nvidia-smi")
        if exe is None:
            return self
        fd, self._path = tempfile.mkstemp(prefix="mf_clocks_", suffix=".csv")
        os.close(fd)
        out = open(self._path, "w")
        self._proc = subprocess.Popen(
            [exe, f"--query-gpu={_QUERY}", "--format=csv,noheader,nounits", "-i", str(self.gpu_index), "-lms", str(self.period_ms)],
            stdout=out, stderr=subprocess.DEVNULL,
        )
        out.close()
        return self

    def __exit__(self, *exc) -> None:
        if self._proc is not None:
            self._proc.terminate()  # the exact child we started
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()

    def summary(self) -> Dict:
        rows: List[List[str]] = []
        if self._path and os.path.exists(self._path):
            with open(self._path) as f:
                for line in f:
                    parts = [p.strip() for p in line.split(",")]
                    if len(parts) >= 9:
                        rows.append(parts)
            os.unlink(self._path)
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm, smax, power = [], [], []
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            try:
                sm.append(float(r[1]))
                smax.append(float(r[2]))
                power.append(float(r[3]))
            except ValueError:
                continue
            for name, val in zip(names, r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        # "Under load" = samples in the upper half of the power range seen; falls back to all samples.
        lo, hi = min(power), max(power)
        loaded = [s for s, p in zip(sm, power) if p >= lo + 0.5 * (hi - lo)] or sm
        return {
            "sm_mhz": statistics.median(loaded),
            "sm_max_mhz": max(smax),
            "power_w_max": hi,
            "reasons": sorted(reasons),
            "samples": len(sm),
        }


def device_time_ms(fn: Callable[[], None], iters: int, stream=None) -> float:
    """Total device time of ``iters`` calls of fn, CUDA events on the launching stream, synchronized on both sides."""
    import torch

    stream = stream or torch.cuda.current_stream()
    start = torch.cuda.Event(enable_timing=True)
    end = torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record(stream)
    for _ in range(iters):
        fn()
    end.record(stream)
    torch.cuda.synchronize()
    return start.elapsed_time(end)


_flush_buf = None


def flush_l2(nbytes: int = 256 << 20) -> None:
    """Writes a buffer larger than the 126 MB L2 so that the next timed iteration starts cold."""
    import torch

    global _flush_buf
    if _flush_buf is None or _flush_buf.numel() < nbytes:
        _flush_buf = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    _flush_buf.fill_(1)
