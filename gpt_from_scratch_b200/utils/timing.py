"""Device-side timing helpers: CUDA-event timers whose result is the maximum over ranks,
and a sampler of SM clocks / throttle reasons that runs while a region is being timed."""
from __future__ import annotations

import statistics
import subprocess
import threading
import time

import torch
import torch.distributed as dist


class CudaTimer:
    """``with CudaTimer() as t: ...`` then ``t.ms`` (synchronises on exit)."""

    def __enter__(self):
        self.e0 = torch.cuda.Event(enable_timing=True)
        self.e1 = torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        self.e0.record()
        return self

    def __exit__(self, *exc):
        self.e1.record()
        torch.cuda.synchronize()
        self.ms = self.e0.elapsed_time(self.e1)
        return False


def max_over_ranks(value: float, device: torch.device) -> float:
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        t = torch.tensor([value], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())
    return float(value)


class ClockSampler:
    """Samples ``nvidia-smi`` SM clocks and throttle reasons of one GPU every 200 ms in a
    background thread (read-only queries; nothing is changed on the device)."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int = 0):
        self.gpu_index = gpu_index
        self.samples: list[list[str]] = []
        self._proc = None
        self._thread = None

    def start(self):
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except (FileNotFoundError, OSError):
            self._proc = None
            return self

        def pump():
            for line in self._proc.stdout:
                parts = [p.strip() for p in line.strip().split(",")]
                if len(parts) >= 7:
                    self.samples.append(parts)
        self._thread = threading.Thread(target=pump, daemon=True)
        self._thread.start()
        return self

    def stop(self) -> dict:
        if self._proc is not None:
            time.sleep(0.05)
            self._proc.terminate()
            try:
                self._proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self._proc.kill()
        sm, reasons, sm_max, power = [], set(), None, []
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                sm_max = float(s[1])
                power.append(float(s[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": sm_max,
                "reasons": sorted(reasons), "samples": len(sm),
                "power_w_max": max(power) if power else None}
