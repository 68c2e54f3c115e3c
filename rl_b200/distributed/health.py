"""Failure detection on the host: heartbeats between ranks, a stall watchdog, and the per-shard health state machine
of a generation fleet.

* :class:`Heartbeat` -- every rank bumps a counter in a shared key-value store (``torch.distributed.TCPStore`` or any
  object with ``set`` / ``get``) from a daemon thread; :meth:`Heartbeat.dead_peers` lists ranks whose counter has not
  moved within the timeout. Ranks consult it *between* steps, before their next collective, so that a lost peer shows
  up as an exception on the host instead of a hung kernel.
* :class:`StallWatchdog` -- raises / calls back when a training loop has not reported progress for too long
  (nemo_rl/algorithms/single_controller.py:1223).
* :class:`HealthTracker` -- HEALTHY -> SUSPECT -> DEAD -> RESTARTING, plus STALE (weights behind) and RETIRED, driven
  by reported successes / failures and probe results; :meth:`select` picks the shards that may serve
  (nemo_rl/models/generation/fleet_health.py:43-57, :95-119, :122, :373).
Nothing here touches a GPU: failures are injected in tests by dropping heartbeats, raising in host code or letting a
rank exit between steps.
"""

from __future__ import annotations

import enum
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Optional


class DictStore:
    """In-process stand-in for a TCPStore (tests, single-process runs)."""

    def __init__(self):
        self._d: dict[str, bytes] = {}
        self._lock = threading.Lock()

    def set(self, k: str, v) -> None:
        with self._lock:
            self._d[k] = v if isinstance(v, bytes) else str(v).encode()

    def get(self, k: str) -> bytes:
        with self._lock:
            return self._d.get(k, b"")


class Heartbeat:
    def __init__(self, store, rank: int, world: int, interval_s: float = 1.0, timeout_s: float = 10.0, prefix: str = "hb",
                 clock: Callable[[], float] = time.monotonic):
        self.store, self.rank, self.world = store, rank, world
        self.interval_s, self.timeout_s, self.prefix, self.clock = interval_s, timeout_s, prefix, clock
        self._count = 0
        self._seen: dict[int, tuple[bytes, float]] = {}
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    def beat(self) -> None:
        self._count += 1
        self.store.set(f"{self.prefix}/{self.rank}", str(self._count))

    def start(self) -> "Heartbeat":
        self.beat()
        self._thread = threading.Thread(target=self._run, daemon=True, name=f"heartbeat-{self.rank}")
        self._thread.start()
        return self

    def _run(self) -> None:
        while not self._stop.wait(self.interval_s):
            try:
                self.beat()
            except Exception:
                return  # the store is gone: the job is shutting down

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval_s + 1)

    def leave(self) -> None:
        """Announces an orderly departure (between steps): peers see it at their next check, without a timeout."""
        self.stop()
        self.store.set(f"{self.prefix}/{self.rank}", "left")

    def dead_peers(self) -> list[int]:
        """Ranks whose heartbeat counter has not changed for ``timeout_s`` (a rank never seen counts from first poll)."""
        now = self.clock()
        dead = []
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                v = self.store.get(f"{self.prefix}/{r}")
            except Exception:
                v = b""
            if v == b"left":
                dead.append(r)
                continue
            last = self._seen.get(r)
            if last is None or last[0] != v:
                self._seen[r] = (v, now)
            elif now - last[1] > self.timeout_s:
                dead.append(r)
        return dead

    def check(self) -> None:
        dead = self.dead_peers()
        if dead:
            raise PeerLostError(f"rank {self.rank}: no heartbeat from ranks {dead} for {self.timeout_s:.0f} s")


class PeerLostError(RuntimeError):
    pass


class StallWatchdog:
    """``progress()`` must be called at least every ``timeout_s``; otherwise ``on_stall`` runs once (default: record)."""

    def __init__(self, timeout_s: float, on_stall: Optional[Callable[[float], None]] = None, poll_s: float = 1.0,
                 clock: Callable[[], float] = time.monotonic):
        self.timeout_s, self.on_stall, self.poll_s, self.clock = timeout_s, on_stall, poll_s, clock
        self._last = clock()
        self.stalled = False
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    def progress(self) -> None:
        self._last = self.clock()
        self.stalled = False

    def poll(self) -> bool:
        idle = self.clock() - self._last
        if idle > self.timeout_s and not self.stalled:
            self.stalled = True
            if self.on_stall is not None:
                self.on_stall(idle)
        return self.stalled

    def start(self) -> "StallWatchdog":
        def run():
            while not self._stop.wait(self.poll_s):
                self.poll()

        self._thread = threading.Thread(target=run, daemon=True, name="stall-watchdog")
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()


# ---------------------------------------------------------------------------------------------- fleet health
class ShardState(enum.Enum):
    HEALTHY = "healthy"
    SUSPECT = "suspect"
    DEAD = "dead"
    RESTARTING = "restarting"
    STALE = "stale"        # alive but serving weights older than allowed
    RETIRED = "retired"    # removed from the fleet for good


@dataclass
class HealthPolicy:
    suspect_after_failures: int = 1     # consecutive failures before HEALTHY -> SUSPECT
    dead_after_failures: int = 3        # consecutive failures before -> DEAD
    recover_after_successes: int = 2    # consecutive successes before SUSPECT -> HEALTHY
    max_restarts: int = 3               # restarts before a shard is RETIRED
    max_weight_lag: int = 1             # weight versions a shard may be behind before it is STALE
    min_healthy_fraction: float = 0.5   # below this the fleet is not serviceable


@dataclass
class _Shard:
    state: ShardState = ShardState.HEALTHY
    failures: int = 0
    successes: int = 0
    restarts: int = 0
    weight_version: int = 0
    last_error: str = ""
    history: list = field(default_factory=list)


class HealthTracker:
    def __init__(self, num_shards: int, policy: Optional[HealthPolicy] = None):
        self.policy = policy or HealthPolicy()
        self.shards = {i: _Shard() for i in range(num_shards)}
        self.current_weight_version = 0
        self._lock = threading.Lock()

    def _set(self, i: int, st: ShardState, why: str = "") -> None:
        s = self.shards[i]
        if s.state != st:
            s.history.append((s.state, st, why))
            s.state = st

    def report_success(self, i: int) -> ShardState:
        with self._lock:
            s = self.shards[i]
            if s.state in (ShardState.DEAD, ShardState.RETIRED, ShardState.RESTARTING):
                return s.state
            s.failures, s.successes = 0, s.successes + 1
            if s.state == ShardState.SUSPECT and s.successes >= self.policy.recover_after_successes:
                self._set(i, ShardState.HEALTHY, "recovered")
            return s.state

    def report_failure(self, i: int, error: str = "", fatal: bool = False) -> ShardState:
        with self._lock:
            s = self.shards[i]
            if s.state in (ShardState.RETIRED, ShardState.DEAD):
                return s.state
            s.failures, s.successes, s.last_error = s.failures + 1, 0, error
            if fatal or s.failures >= self.policy.dead_after_failures:
                self._set(i, ShardState.DEAD, error)
            elif s.failures >= self.policy.suspect_after_failures and s.state == ShardState.HEALTHY:
                self._set(i, ShardState.SUSPECT, error)
            return s.state

    def begin_restart(self, i: int) -> ShardState:
        with self._lock:
            s = self.shards[i]
            if s.state != ShardState.DEAD:
                return s.state
            if s.restarts >= self.policy.max_restarts:
                self._set(i, ShardState.RETIRED, "restart budget spent")
            else:
                s.restarts += 1
                self._set(i, ShardState.RESTARTING, "restart")
            return s.state

    def finish_restart(self, i: int, ok: bool, weight_version: Optional[int] = None) -> ShardState:
        with self._lock:
            s = self.shards[i]
            if s.state != ShardState.RESTARTING:
                return s.state
            if ok:
                s.failures = s.successes = 0
                s.weight_version = self.current_weight_version if weight_version is None else weight_version
                self._set(i, ShardState.HEALTHY if self.current_weight_version - s.weight_version <= self.policy.max_weight_lag
                          else ShardState.STALE, "restarted")
            else:
                self._set(i, ShardState.DEAD, "restart failed")
            return s.state

    def set_weight_version(self, version: int, updated_shards: Optional[list[int]] = None) -> None:
        """The trainer published ``version``; ``updated_shards`` received it (default: all serviceable shards)."""
        with self._lock:
            self.current_weight_version = version
            for i, s in self.shards.items():
                if updated_shards is None or i in updated_shards:
                    if s.state in (ShardState.HEALTHY, ShardState.SUSPECT, ShardState.STALE):
                        s.weight_version = version
                        if s.state == ShardState.STALE:
                            self._set(i, ShardState.HEALTHY, "weights caught up")
                elif s.state == ShardState.HEALTHY and version - s.weight_version > self.policy.max_weight_lag:
                    self._set(i, ShardState.STALE, f"weights {version - s.weight_version} versions behind")

    def state(self, i: int) -> ShardState:
        return self.shards[i].state

    def select(self, include_suspect: bool = True) -> list[int]:
        """Shards that may take requests, healthy ones first."""
        with self._lock:
            ok = [i for i, s in self.shards.items() if s.state == ShardState.HEALTHY]
            if include_suspect:
                ok += [i for i, s in self.shards.items() if s.state == ShardState.SUSPECT]
            return ok

    def serviceable(self) -> bool:
        alive = [s for s in self.shards.values() if s.state != ShardState.RETIRED]
        healthy = len(self.select(include_suspect=True))
        return bool(alive) and healthy / len(self.shards) >= self.policy.min_healthy_fraction

    def summary(self) -> dict[str, int]:
        out: dict[str, int] = {}
        for s in self.shards.values():
            out[s.state.value] = out.get(s.state.value, 0) + 1
        return out
