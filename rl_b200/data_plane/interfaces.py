"""Data plane: a key-addressed store of per-sample tensor records between rollout producers and training consumers.

Producers ``put`` one record per sample (a dict of named fields: tensors of any length, scalars, strings or small python
objects); consumers ask for the fields they need of the keys they were assigned. Only keys and small metadata travel
through the controller; the payload moves producer -> store -> consumer once. The contract mirrors
nemo_rl/data_plane/interfaces.py:92-248 (client), with in-process and TCP-store adapters in place of
TransferQueue / Mooncake.
"""

from __future__ import annotations

import abc
from dataclasses import dataclass, field
from typing import Any, Iterable, Optional, Sequence


@dataclass
class SampleMeta:
    """What the controller knows about a stored sample without touching its payload."""
    key: str
    num_tokens: int = 0
    weight_version: int = 0
    group: Optional[str] = None          # samples of one prompt share a group (advantages are computed per group)
    fields: tuple = ()
    extra: dict = field(default_factory=dict)


class DataPlaneClient(abc.ABC):
    @abc.abstractmethod
    def put(self, key: str, record: dict[str, Any], meta: Optional[SampleMeta] = None) -> SampleMeta: ...

    @abc.abstractmethod
    def get(self, keys: Sequence[str], fields: Optional[Iterable[str]] = None) -> list[dict[str, Any]]: ...

    @abc.abstractmethod
    def update(self, key: str, record: dict[str, Any]) -> None:
        """Adds or replaces fields of a stored sample (log-probabilities and advantages are written back this way)."""

    @abc.abstractmethod
    def delete(self, keys: Sequence[str]) -> int: ...

    @abc.abstractmethod
    def list_meta(self, prefix: str = "") -> list[SampleMeta]: ...

    def put_batch(self, keys: Sequence[str], records: Sequence[dict[str, Any]], metas: Optional[Sequence[SampleMeta]] = None) -> list[SampleMeta]:
        return [self.put(k, r, metas[i] if metas else None) for i, (k, r) in enumerate(zip(keys, records))]

    def stats(self) -> dict[str, float]:
        return {}

    def close(self) -> None:
        pass
