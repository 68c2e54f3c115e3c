"""Cross-process adapter over a ``torch.distributed.TCPStore``: any rank (or a controller outside the training world) puts
and gets records by key through the store's server. Payloads are chunked below the store's comfortable value size."""

from __future__ import annotations

import pickle
from typing import Any, Iterable, Optional, Sequence

from ..codec import decode_record, encode_record, record_fields
from ..interfaces import DataPlaneClient, SampleMeta

_CHUNK = 8 << 20


class TCPStoreDataPlane(DataPlaneClient):
    def __init__(self, store, namespace: str = "dp"):
        """``store``: a ``TCPStore`` (or anything with set/get/add/delete_key, such as the in-memory test double)."""
        self.store, self.ns = store, namespace

    def _k(self, key: str, part: str) -> str:
        return f"{self.ns}/{key}/{part}"

    def put(self, key, record, meta=None):
        buf = encode_record(record)
        n = max(1, (len(buf) + _CHUNK - 1) // _CHUNK)
        for i in range(n):
            self.store.set(self._k(key, f"c{i}"), buf[i * _CHUNK : (i + 1) * _CHUNK])
        m = meta or SampleMeta(key)
        m.key, m.fields = key, tuple(record_fields(buf))
        self.store.set(self._k(key, "meta"), pickle.dumps((n, m)))
        idx = self.store.add(f"{self.ns}/__count__", 1)          # append-only index of keys
        self.store.set(f"{self.ns}/__index__/{idx}", key.encode())
        return m

    def _has(self, full_key: str) -> bool:
        chk = getattr(self.store, "check", None)     # a TCPStore get() on a missing key would wait for its timeout
        if chk is not None:
            return bool(chk([full_key]))
        try:
            self.store.get(full_key)
            return True
        except Exception:
            return False

    def _load(self, key: str) -> bytes:
        if not self._has(self._k(key, "meta")):
            raise KeyError(key)
        n, _ = pickle.loads(self.store.get(self._k(key, "meta")))
        return b"".join(bytes(self.store.get(self._k(key, f"c{i}"))) for i in range(n))

    def get(self, keys: Sequence[str], fields: Optional[Iterable[str]] = None) -> list[dict[str, Any]]:
        want = set(fields) | {"__jagged__"} if fields is not None else None
        return [decode_record(self._load(k), want) for k in keys]

    def update(self, key, record):
        cur = decode_record(self._load(key))
        cur.update(record)
        _, m = pickle.loads(self.store.get(self._k(key, "meta")))
        self.put(key, cur, m)

    def delete(self, keys):
        n = 0
        for k in keys:
            if not self._has(self._k(k, "meta")):
                continue
            cnt, _ = pickle.loads(self.store.get(self._k(k, "meta")))
            for i in range(cnt):
                self.store.delete_key(self._k(k, f"c{i}"))
            self.store.delete_key(self._k(k, "meta"))
            n += 1
        return n

    def list_meta(self, prefix: str = ""):
        total = self.store.add(f"{self.ns}/__count__", 0)
        seen, out = set(), []
        for i in range(1, total + 1):
            k = bytes(self.store.get(f"{self.ns}/__index__/{i}")).decode()
            if k in seen or not k.startswith(prefix):
                continue
            seen.add(k)
            if self._has(self._k(k, "meta")):   # not deleted since
                out.append(pickle.loads(self.store.get(self._k(k, "meta")))[1])
        return out
