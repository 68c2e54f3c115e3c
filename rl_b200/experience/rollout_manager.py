"""Rollout manager: runs per-sample (or per-group) rollout jobs with a retry policy, deadlines and failure accounting
(nemo_rl/experience/rollout_manager.py:74-139, :351, :729).

Infrastructure failures are retried (optionally on another shard chosen through a :class:`HealthTracker`) with
exponential back-off until ``max_attempts`` or the deadline; data failures are not retried: the sample comes back
masked (``loss_multiplier = 0``) so the batch shape is preserved. ``max_failed_fraction`` bounds how much of a batch
may be lost before the step is abandoned (async GRPO's ``max_generation_failures``).
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Any, Callable, Optional, Sequence

from rl_b200.experience.failures import DeadlineExceeded, FailureKind, FailureRecord, InfraFailure, classify


@dataclass
class RetryPolicy:
    max_attempts: int = 3
    backoff_s: float = 0.0
    backoff_factor: float = 2.0
    deadline_s: Optional[float] = None          # wall-clock budget of one job including retries
    max_failed_fraction: float = 0.25           # of the jobs of one run() call
    retry_data_failures: bool = False


@dataclass
class JobResult:
    index: int
    value: Any = None
    ok: bool = False
    attempts: int = 0
    failures: list[FailureRecord] = field(default_factory=list)

    @property
    def kind(self) -> Optional[FailureKind]:
        return None if self.ok or not self.failures else self.failures[-1].kind


class TooManyFailures(InfraFailure):
    pass


class RolloutManager:
    def __init__(self, policy: Optional[RetryPolicy] = None, health=None, clock: Callable[[], float] = time.monotonic,
                 sleep: Callable[[float], None] = time.sleep):
        self.policy = policy or RetryPolicy()
        self.health = health
        self.clock, self.sleep = clock, sleep
        self.stats = dict(jobs=0, retries=0, infra_failures=0, data_failures=0, abandoned=0)

    def _pick_shard(self, attempt: int, avoid: set) -> Optional[int]:
        if self.health is None:
            return None
        cands = [s for s in self.health.select() if s not in avoid] or self.health.select()
        if not cands:
            raise InfraFailure("no serviceable generation shard")
        return cands[attempt % len(cands)]

    def run_one(self, index: int, fn: Callable[..., Any], item: Any) -> JobResult:
        p = self.policy
        res = JobResult(index)
        t0 = self.clock()
        delay = p.backoff_s
        avoid: set = set()
        while res.attempts < p.max_attempts:
            if p.deadline_s is not None and self.clock() - t0 > p.deadline_s:
                res.failures.append(FailureRecord(FailureKind.INFRA, "deadline exceeded", res.attempts, index))
                break
            res.attempts += 1
            shard = self._pick_shard(res.attempts - 1, avoid)
            try:
                res.value = fn(item) if shard is None else fn(item, shard)
                res.ok = True
                if self.health is not None and shard is not None:
                    self.health.report_success(shard)
                return res
            except BaseException as e:  # noqa: BLE001 - every failure is classified
                if isinstance(e, (KeyboardInterrupt, SystemExit)):
                    raise
                kind = classify(e)
                res.failures.append(FailureRecord(kind, f"{type(e).__name__}: {e}", res.attempts, index, shard))
                if kind == FailureKind.INFRA:
                    self.stats["infra_failures"] += 1
                    if self.health is not None and shard is not None:
                        self.health.report_failure(shard, str(e))
                        avoid.add(shard)
                else:
                    self.stats["data_failures"] += 1
                    if not p.retry_data_failures:
                        break
                if res.attempts < p.max_attempts:
                    self.stats["retries"] += 1
                    if delay > 0:
                        self.sleep(delay)
                        delay *= p.backoff_factor
        return res

    def run(self, fn: Callable[..., Any], items: Sequence[Any]) -> list[JobResult]:
        """Runs ``fn(item)`` (or ``fn(item, shard)`` with a health tracker) for every item. Raises
        :class:`TooManyFailures` when more than ``max_failed_fraction`` of the jobs ended without a result."""
        out = []
        for i, it in enumerate(items):
            self.stats["jobs"] += 1
            out.append(self.run_one(i, fn, it))
        failed = sum(1 for r in out if not r.ok)
        self.stats["abandoned"] += failed
        if items and failed / len(items) > self.policy.max_failed_fraction:
            raise TooManyFailures(f"{failed}/{len(items)} rollout jobs failed (limit {self.policy.max_failed_fraction:.0%})")
        return out
