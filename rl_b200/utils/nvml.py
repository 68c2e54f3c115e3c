"""Read-only NVML helpers: device identity, memory, clocks and throttle reasons.

Everything here *reads* device state; nothing sets clocks, power limits, persistence or compute mode. ``handle`` may be
any object with the ``pynvml`` function names, which is how the tests run against a fake library. Role of
nemo_rl/utils/nvml.py (device-uuid lookup for CUDA-IPC refit, free-memory queries).
"""

from __future__ import annotations

import contextlib
from typing import Any, Optional

THROTTLE_BITS = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x10: "sync_boost",
                 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}


@contextlib.contextmanager
def nvml_context(lib: Any = None):
    """Initialises NVML for the duration of the block and always shuts it down again."""
    if lib is None:
        import pynvml as lib
    lib.nvmlInit()
    try:
        yield lib
    finally:
        lib.nvmlShutdown()


def _s(x) -> str:
    return x.decode() if isinstance(x, bytes) else str(x)


def device_id_to_physical(device_idx: int, visible: Optional[str] = None) -> int:
    """Maps a process-local CUDA ordinal to the NVML index through ``CUDA_VISIBLE_DEVICES`` (numeric entries only)."""
    import os

    vis = os.environ.get("CUDA_VISIBLE_DEVICES") if visible is None else visible
    if not vis:
        return device_idx
    ids = [v.strip() for v in vis.split(",") if v.strip()]
    if device_idx >= len(ids):
        raise ValueError(f"device {device_idx} is not among the {len(ids)} visible devices")
    return int(ids[device_idx]) if ids[device_idx].isdigit() else device_idx


def get_device_uuid(device_idx: int, lib: Any = None) -> str:
    with nvml_context(lib) as n:
        return _s(n.nvmlDeviceGetUUID(n.nvmlDeviceGetHandleByIndex(device_id_to_physical(device_idx))))


def get_free_memory_bytes(device_idx: int, lib: Any = None) -> int:
    with nvml_context(lib) as n:
        return int(n.nvmlDeviceGetMemoryInfo(n.nvmlDeviceGetHandleByIndex(device_id_to_physical(device_idx))).free)


def decode_throttle_reasons(mask: int) -> list[str]:
    return [name for bit, name in THROTTLE_BITS.items() if mask & bit and name != "gpu_idle"]


def snapshot(device_idx: int, lib: Any = None) -> dict:
    """One reading of what a benchmark has to record beside its number: clocks, power, memory, throttle reasons."""
    with nvml_context(lib) as n:
        h = n.nvmlDeviceGetHandleByIndex(device_id_to_physical(device_idx))
        mem = n.nvmlDeviceGetMemoryInfo(h)
        out = dict(name=_s(n.nvmlDeviceGetName(h)), uuid=_s(n.nvmlDeviceGetUUID(h)), memory_used=int(mem.used), memory_total=int(mem.total),
                   sm_mhz=int(n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_SM)), sm_max_mhz=int(n.nvmlDeviceGetMaxClockInfo(h, n.NVML_CLOCK_SM)),
                   power_w=n.nvmlDeviceGetPowerUsage(h) / 1000.0)
        try:
            out["reasons"] = decode_throttle_reasons(int(n.nvmlDeviceGetCurrentClocksEventReasons(h)))
        except Exception:
            out["reasons"] = decode_throttle_reasons(int(n.nvmlDeviceGetCurrentClocksThrottleReasons(h)))
        return out
