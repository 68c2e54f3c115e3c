"""Profiling hooks and NVML telemetry against a fake backend (no GPU setting is ever changed)."""

import types

import pytest

from rl_b200.utils import profiling as P


def test_step_range_capture(monkeypatch):
    calls = []
    monkeypatch.setenv("RLB_PROFILE_STEP_RANGE", "2:4")
    P._state["active"] = False
    out = [P.maybe_gpu_profile_step(s, 0, lambda: calls.append("start"), lambda: calls.append("stop")) for s in range(6)]
    assert out == [None, None, "start", None, "stop", None] and calls == ["start", "stop"]
    assert P.maybe_gpu_profile_step(2, 1, lambda: calls.append("x"), None) is None  # rank 1 is not selected by default
    monkeypatch.setenv("RLB_PROFILE_STEP_RANGE", "5:3")
    with pytest.raises(ValueError):
        P.maybe_gpu_profile_step(0)


def test_nvml_reads_only():
    touched = []

    class Fake:
        NVML_CLOCK_SM, NVML_TEMPERATURE_GPU = 1, 0

        def nvmlInit(self): touched.append("init")
        def nvmlShutdown(self): touched.append("shutdown")
        def nvmlDeviceGetHandleByIndex(self, i): return i
        def nvmlDeviceGetCurrentClocksEventReasons(self, h): return 0x4 | 0x1
        def nvmlDeviceGetUtilizationRates(self, h): return types.SimpleNamespace(gpu=97, memory=40)
        def nvmlDeviceGetMemoryInfo(self, h): return types.SimpleNamespace(used=90 * 2**30, total=180 * 2**30)
        def nvmlDeviceGetClockInfo(self, h, k): return 1755
        def nvmlDeviceGetMaxClockInfo(self, h, k): return 1965
        def nvmlDeviceGetPowerUsage(self, h): return 987000
        def nvmlDeviceGetTemperature(self, h, k): return 61

        def __getattr__(self, name):  # any setter would land here
            raise AssertionError(f"unexpected NVML call {name}")

    n = P.Nvml(Fake())
    s = n.sample(0)
    assert s["sm_mhz"] == 1755 and s["sm_max_mhz"] == 1965 and s["reasons"] == ["sw_power_cap"] and s["power_w"] == 987.0
    n.shutdown()
    assert touched == ["init", "shutdown"]


def test_memory_tracker_and_nvtx_on_cpu():
    t = P.MemoryTracker()
    t.snapshot("after_generation")
    assert "after_generation/peak_gb" in t.as_metrics()

    @P.wrap_with_nvtx_name("phase")
    def f(x):
        return x + 1

    assert f(1) == 2
