"""Nested named timers with reductions, a thread-safe variant and a wall-clock deadline checker.

Names use ``/`` for nesting (``prepare_for_generation/total``); the algorithms log them under ``timing/train/*`` with
the same names the reference uses (nemo_rl/utils/timer.py:27-476), so downstream performance scripts carry over.
"""

from __future__ import annotations

import threading
import time
from collections import defaultdict
from contextlib import contextmanager
from typing import Callable, Optional, Sequence

import numpy as np

_REDUCTIONS: dict[str, Callable[[Sequence[float]], float]] = {
    "mean": lambda x: float(np.mean(x)),
    "median": lambda x: float(np.median(x)),
    "min": lambda x: float(np.min(x)),
    "max": lambda x: float(np.max(x)),
    "std": lambda x: float(np.std(x)),
    "sum": lambda x: float(np.sum(x)),
    "count": lambda x: float(len(x)),
}


class Timer:
    def __init__(self):
        self._timers: dict[str, list[float]] = defaultdict(list)
        self._starts: dict[str, float] = {}

    def start(self, label: str) -> None:
        if label in self._starts:
            raise ValueError(f"timer '{label}' is already running")
        self._starts[label] = time.perf_counter()

    def stop(self, label: str) -> float:
        if label not in self._starts:
            raise ValueError(f"timer '{label}' was not started")
        dt = time.perf_counter() - self._starts.pop(label)
        self._timers[label].append(dt)
        return dt

    @contextmanager
    def time(self, label: str):
        self.start(label)
        try:
            yield
        finally:
            self.stop(label)

    def get_elapsed(self, label: str) -> list[float]:
        return list(self._timers[label])

    def get_latest_elapsed(self, label: str) -> float:
        return self._timers[label][-1]

    def reduce(self, label: str, operation: str = "mean") -> float:
        if operation not in _REDUCTIONS:
            raise ValueError(f"unknown reduction '{operation}' ({sorted(_REDUCTIONS)})")
        if not self._timers[label]:
            raise KeyError(f"timer '{label}' has no measurements")
        return _REDUCTIONS[operation](self._timers[label])

    def get_timing_metrics(self, reduction_op: str | dict[str, str] = "mean") -> dict[str, float]:
        out = {}
        for label in self._timers:
            op = reduction_op.get(label, "mean") if isinstance(reduction_op, dict) else reduction_op
            out[label] = self.reduce(label, op)
        return out

    def reset(self, label: Optional[str] = None) -> None:
        if label is None:
            self._timers.clear()
            self._starts.clear()
        else:
            self._timers.pop(label, None)
            self._starts.pop(label, None)


class ThreadSafeTimer(Timer):
    """Timer whose running set is per-thread and whose measurements are guarded by a lock."""

    def __init__(self):
        super().__init__()
        self._lock = threading.Lock()
        self._local = threading.local()

    def start(self, label: str) -> None:
        starts = getattr(self._local, "starts", None)
        if starts is None:
            starts = self._local.starts = {}
        if label in starts:
            raise ValueError(f"timer '{label}' is already running on this thread")
        starts[label] = time.perf_counter()

    def stop(self, label: str) -> float:
        starts = getattr(self._local, "starts", {})
        if label not in starts:
            raise ValueError(f"timer '{label}' was not started on this thread")
        dt = time.perf_counter() - starts.pop(label)
        with self._lock:
            self._timers[label].append(dt)
        return dt


class TimeoutChecker:
    """Says when a checkpoint must be forced before a wall-clock limit (``checkpoint_must_save_by``).

    ``timeout``: "DD:HH:MM:SS" (or fewer fields) or seconds; None disables. With ``fit_last_save_time`` the checker
    keeps a running mean of iteration time and fires when one more iteration would cross the limit."""

    def __init__(self, timeout: Optional[str | float] = None, fit_last_save_time: bool = False):
        self.start_time = time.time()
        self.fit = fit_last_save_time
        self.iter_times: list[float] = []
        self.last = self.start_time
        self.timeout = self._parse(timeout)

    @staticmethod
    def _parse(t) -> Optional[float]:
        if t is None:
            return None
        if isinstance(t, (int, float)):
            return float(t)
        parts = [int(p) for p in str(t).split(":")]
        while len(parts) < 4:
            parts.insert(0, 0)
        d, h, m, s = parts
        return float(((d * 24 + h) * 60 + m) * 60 + s)

    def mark_iteration(self) -> None:
        now = time.time()
        self.iter_times.append(now - self.last)
        self.last = now

    def start_iterations(self) -> None:
        self.last = time.time()

    def check_save(self) -> bool:
        if self.timeout is None:
            return False
        elapsed = time.time() - self.start_time
        margin = float(np.mean(self.iter_times)) if (self.fit and self.iter_times) else 0.0
        return elapsed + margin >= self.timeout
