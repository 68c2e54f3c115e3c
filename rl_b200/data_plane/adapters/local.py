"""In-process store (one controller process, or tests): records stay encoded so that the byte accounting and the field
selection behave like the networked adapter."""

from __future__ import annotations

import threading
from typing import Any, Iterable, Optional, Sequence

from ..codec import decode_record, encode_record, record_fields
from ..interfaces import DataPlaneClient, SampleMeta


class LocalDataPlane(DataPlaneClient):
    def __init__(self, capacity_bytes: Optional[int] = None):
        self._data: dict[str, bytes] = {}
        self._meta: dict[str, SampleMeta] = {}
        self._lock = threading.Lock()
        self.capacity = capacity_bytes
        self._stats = dict(puts=0, gets=0, bytes_in=0, bytes_out=0, deletes=0)

    def _bytes(self) -> int:
        return sum(len(v) for v in self._data.values())

    def put(self, key, record, meta=None):
        buf = encode_record(record)
        with self._lock:
            if self.capacity is not None and self._bytes() + len(buf) > self.capacity:
                raise MemoryError(f"data plane full: {self._bytes()} + {len(buf)} > {self.capacity} bytes")
            self._data[key] = buf
            m = meta or SampleMeta(key)
            m.key, m.fields = key, tuple(record_fields(buf))
            self._meta[key] = m
            self._stats["puts"] += 1
            self._stats["bytes_in"] += len(buf)
        return m

    def get(self, keys: Sequence[str], fields: Optional[Iterable[str]] = None) -> list[dict[str, Any]]:
        want = set(fields) | {"__jagged__"} if fields is not None else None
        out = []
        with self._lock:
            bufs = [self._data[k] for k in keys]     # KeyError names the missing key
            self._stats["gets"] += len(bufs)
            self._stats["bytes_out"] += sum(len(b) for b in bufs)
        for b in bufs:
            out.append(decode_record(b, want))
        return out

    def update(self, key, record):
        with self._lock:
            cur = decode_record(self._data[key])
        cur.update(record)
        buf = encode_record(cur)
        with self._lock:
            self._data[key] = buf
            self._meta[key].fields = tuple(record_fields(buf))

    def delete(self, keys):
        n = 0
        with self._lock:
            for k in keys:
                if self._data.pop(k, None) is not None:
                    self._meta.pop(k, None)
                    n += 1
            self._stats["deletes"] += n
        return n

    def list_meta(self, prefix: str = ""):
        with self._lock:
            return [m for k, m in self._meta.items() if k.startswith(prefix)]

    def stats(self):
        with self._lock:
            return dict(self._stats, resident_bytes=self._bytes(), resident_samples=len(self._data))
