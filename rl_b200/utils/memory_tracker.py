"""Stage-by-stage memory bookkeeping (host RSS and device allocator), as nemo_rl/utils/memory_tracker.py does for the
driver process: ``snapshot_start_of_stage`` at every phase boundary, a table at the end."""

from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Optional


def host_rss_bytes() -> int:
    try:
        import psutil

        return int(psutil.Process(os.getpid()).memory_info().rss)
    except Exception:
        with open("/proc/self/statm") as f:
            return int(f.read().split()[1]) * os.sysconf("SC_PAGE_SIZE")


@dataclass
class MemoryPoint:
    stage: str
    host_rss: int
    device_allocated: int = 0
    device_reserved: int = 0
    device_peak: int = 0
    after_host_rss: Optional[int] = None
    after_device_allocated: Optional[int] = None


@dataclass
class MemoryTracker:
    points: list = field(default_factory=list)

    def _device(self):
        import torch

        if not torch.cuda.is_available():
            return 0, 0, 0
        return torch.cuda.memory_allocated(), torch.cuda.memory_reserved(), torch.cuda.max_memory_allocated()

    def snapshot_start_of_stage(self, stage: str) -> MemoryPoint:
        if self.points:
            last = self.points[-1]
            last.after_host_rss, last.after_device_allocated = host_rss_bytes(), self._device()[0]
        a, r, p = self._device()
        pt = MemoryPoint(stage, host_rss_bytes(), a, r, p)
        self.points.append(pt)
        return pt

    def deltas(self) -> list[dict]:
        out = []
        for p in self.points:
            out.append(dict(stage=p.stage, host_rss_gib=p.host_rss / 2**30, device_allocated_gib=p.device_allocated / 2**30,
                            host_delta_gib=None if p.after_host_rss is None else (p.after_host_rss - p.host_rss) / 2**30,
                            device_delta_gib=None if p.after_device_allocated is None else (p.after_device_allocated - p.device_allocated) / 2**30))
        return out

    def table(self) -> str:
        rows = ["stage                          host GiB   dev GiB   d host   d dev"]
        for d in self.deltas():
            f = lambda v: "     -" if v is None else f"{v:+6.2f}"  # noqa: E731
            rows.append(f"{d['stage'][:30]:30s} {d['host_rss_gib']:8.2f} {d['device_allocated_gib']:9.2f} {f(d['host_delta_gib'])}  {f(d['device_delta_gib'])}")
        return "\n".join(rows)
