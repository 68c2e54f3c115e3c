"""Event statistics of a data-plane client: per-operation counts, bytes and latency, as a wrapper around any client
(nemo_rl/data_plane/observability.py:38-86 keeps the same kind of counters for TransferQueue)."""

from __future__ import annotations

import time
from collections import defaultdict
from typing import Any

from .interfaces import DataPlaneClient


class ObservedDataPlane(DataPlaneClient):
    def __init__(self, inner: DataPlaneClient):
        self.inner = inner
        self.events: dict[str, dict[str, float]] = defaultdict(lambda: dict(calls=0, items=0, seconds=0.0, max_seconds=0.0))

    def _timed(self, op: str, n: int, fn, *a, **k) -> Any:
        t0 = time.perf_counter()
        try:
            return fn(*a, **k)
        finally:
            dt = time.perf_counter() - t0
            e = self.events[op]
            e["calls"] += 1
            e["items"] += n
            e["seconds"] += dt
            e["max_seconds"] = max(e["max_seconds"], dt)

    def put(self, key, record, meta=None):
        return self._timed("put", 1, self.inner.put, key, record, meta)

    def get(self, keys, fields=None):
        return self._timed("get", len(keys), self.inner.get, keys, fields)

    def update(self, key, record):
        return self._timed("update", 1, self.inner.update, key, record)

    def delete(self, keys):
        return self._timed("delete", len(keys), self.inner.delete, keys)

    def list_meta(self, prefix=""):
        return self._timed("list_meta", 1, self.inner.list_meta, prefix)

    def stats(self):
        out = dict(self.inner.stats())
        for op, e in self.events.items():
            for k, v in e.items():
                out[f"{op}_{k}"] = v
        return out

    def close(self):
        self.inner.close()
