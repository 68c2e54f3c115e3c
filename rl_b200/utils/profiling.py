"""Profiling hooks: a step-range capture switch, NVTX ranges, a memory tracker and read-only NVML queries.

* ``RLB_PROFILE_STEP_RANGE=start:stop`` makes :func:`maybe_gpu_profile_step` call ``cudaProfilerStart`` before step
  ``start`` and ``cudaProfilerStop`` before step ``stop`` (run the job under a profiler with
  ``--capture-range=cudaProfilerApi``); ``RLB_PROFILE_RANKS`` (comma list, default ``0``) selects the ranks. This is the
  role of ``NRL_NSYS_PROFILE_STEP_RANGE`` / ``NRL_NSYS_WORKER_PATTERNS`` (nemo_rl/utils/nsys.py:22-110).
* :func:`nvtx_range` / :func:`wrap_with_nvtx_name` tag phases (nemo_rl/utils/nsys.py:113-125).
* :class:`MemoryTracker` records allocator statistics per named stage (nemo_rl/utils/memory_tracker.py).
* :class:`Nvml` reads clocks, power, temperature, utilisation and throttle reasons. It never changes a setting; a fake
  backend can be injected for tests (nemo_rl/utils/nvml.py).
"""

from __future__ import annotations

import contextlib
import functools
import os
from dataclasses import dataclass, field
from typing import Any, Callable, Optional

import torch

_state = {"active": False}


def _range_from_env() -> Optional[tuple[int, int]]:
    v = os.environ.get("RLB_PROFILE_STEP_RANGE") or os.environ.get("NRL_NSYS_PROFILE_STEP_RANGE")
    if not v:
        return None
    a, b = v.split(":")
    a, b = int(a), int(b)
    if not (0 <= a < b):
        raise ValueError(f"profile step range must be start:stop with 0 <= start < stop, got {v!r}")
    return a, b


def _rank_selected(rank: int) -> bool:
    sel = os.environ.get("RLB_PROFILE_RANKS", "0")
    return sel == "all" or str(rank) in [s.strip() for s in sel.split(",")]


def maybe_gpu_profile_step(step: int, rank: int = 0, start: Callable[[], None] = None, stop: Callable[[], None] = None) -> Optional[str]:
    """Call at the top of every step. Returns "start" / "stop" when it toggled the capture, else None."""
    rng = _range_from_env()
    if rng is None or not _rank_selected(rank):
        return None
    start = start or (torch.cuda.profiler.start if torch.cuda.is_available() else (lambda: None))
    stop = stop or (torch.cuda.profiler.stop if torch.cuda.is_available() else (lambda: None))
    if step == rng[0] and not _state["active"]:
        start()
        _state["active"] = True
        return "start"
    if step >= rng[1] and _state["active"]:
        stop()
        _state["active"] = False
        return "stop"
    return None


@contextlib.contextmanager
def nvtx_range(name: str):
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


def wrap_with_nvtx_name(name: str):
    def deco(fn):
        @functools.wraps(fn)
        def inner(*a, **k):
            with nvtx_range(name):
                return fn(*a, **k)

        return inner

    return deco


@dataclass
class MemoryPoint:
    stage: str
    allocated_gb: float
    reserved_gb: float
    peak_gb: float


@dataclass
class MemoryTracker:
    device: Any = None
    points: list[MemoryPoint] = field(default_factory=list)

    def snapshot(self, stage: str) -> MemoryPoint:
        if torch.cuda.is_available():
            a = torch.cuda.memory_allocated(self.device) / 2**30
            r = torch.cuda.memory_reserved(self.device) / 2**30
            p = torch.cuda.max_memory_allocated(self.device) / 2**30
            torch.cuda.reset_peak_memory_stats(self.device)
        else:
            a = r = p = 0.0
        pt = MemoryPoint(stage, a, r, p)
        self.points.append(pt)
        return pt

    def as_metrics(self) -> dict[str, float]:
        out = {}
        for pt in self.points:
            out[f"{pt.stage}/allocated_gb"] = pt.allocated_gb
            out[f"{pt.stage}/peak_gb"] = pt.peak_gb
        return out


class Nvml:
    """Read-only device telemetry. ``backend`` is the ``pynvml`` module (or a fake with the same functions)."""

    THROTTLE_BITS = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x10: "sync_boost",
                     0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}

    def __init__(self, backend=None):
        if backend is None:
            import pynvml as backend  # provided by nvidia-ml-py

        self.nv = backend
        self.nv.nvmlInit()

    def sample(self, index: int = 0) -> dict:
        nv = self.nv
        h = nv.nvmlDeviceGetHandleByIndex(index)
        reasons = int(nv.nvmlDeviceGetCurrentClocksEventReasons(h)) if hasattr(nv, "nvmlDeviceGetCurrentClocksEventReasons") \
            else int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(h))
        util = nv.nvmlDeviceGetUtilizationRates(h)
        mem = nv.nvmlDeviceGetMemoryInfo(h)
        return {
            "sm_mhz": int(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)),
            "sm_max_mhz": int(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)),
            "power_w": nv.nvmlDeviceGetPowerUsage(h) / 1000.0,
            "temperature_c": int(nv.nvmlDeviceGetTemperature(h, nv.NVML_TEMPERATURE_GPU)),
            "gpu_util": int(util.gpu), "mem_util": int(util.memory),
            "mem_used_gb": mem.used / 2**30, "mem_total_gb": mem.total / 2**30,
            "reasons": [name for bit, name in self.THROTTLE_BITS.items() if reasons & bit and name != "gpu_idle"],
        }

    def shutdown(self) -> None:
        try:
            self.nv.nvmlShutdown()
        except Exception:
            pass
