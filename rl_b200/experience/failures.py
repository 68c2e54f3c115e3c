"""Failure taxonomy of rollouts (nemo_rl/experience/failures.py:236): *infrastructure* failures (a generation shard or
an environment worker broke: retry elsewhere, the sample is fine) versus *data* failures (this sample cannot be
processed: malformed tool call, over-long prompt, environment rejected it: do not retry, mask it out)."""

from __future__ import annotations

import asyncio
import enum
from dataclasses import dataclass
from typing import Optional


class FailureKind(enum.Enum):
    INFRA = "infra"
    DATA = "data"


class RolloutFailure(Exception):
    kind = FailureKind.INFRA

    def __init__(self, message: str = "", *, shard: Optional[int] = None, sample_idx: Optional[int] = None):
        super().__init__(message)
        self.shard, self.sample_idx = shard, sample_idx


class InfraFailure(RolloutFailure):
    kind = FailureKind.INFRA


class DataFailure(RolloutFailure):
    kind = FailureKind.DATA


class DeadlineExceeded(InfraFailure):
    pass


@dataclass
class FailureRecord:
    kind: FailureKind
    error: str
    attempt: int
    sample_idx: Optional[int] = None
    shard: Optional[int] = None


_INFRA_TYPES = (ConnectionError, TimeoutError, asyncio.TimeoutError, OSError, MemoryError)
_DATA_TYPES = (ValueError, KeyError, IndexError, UnicodeError, AssertionError)


def classify(exc: BaseException) -> FailureKind:
    """Maps an arbitrary exception onto the taxonomy (explicit RolloutFailure subclasses win)."""
    if isinstance(exc, RolloutFailure):
        return exc.kind
    if isinstance(exc, _INFRA_TYPES):
        return FailureKind.INFRA
    if isinstance(exc, _DATA_TYPES):
        return FailureKind.DATA
    return FailureKind.INFRA
