"""HTTP router in front of several generation servers, with health tracking and failover.

One address for external agents: each request goes to a healthy shard (fewest requests in flight first); a shard that
fails is reported to the :class:`HealthTracker`, the request is retried on another shard, and dead shards are probed in
the background until they answer ``/health`` again. This is the job of the reference's generation router and fleet
health monitor (nemo_rl/models/generation/generation_router.py, fleet_health.py:43-119).
"""

from __future__ import annotations

import threading
import time
from typing import Any, Optional

from rl_b200.distributed.health import HealthPolicy, HealthTracker, ShardState


class NoHealthyShardError(RuntimeError):
    pass


class GenerationRouter:
    def __init__(self, shard_urls: list[str], policy: Optional[HealthPolicy] = None, request_timeout_s: float = 600.0,
                 probe_interval_s: float = 2.0, max_attempts: Optional[int] = None, session=None):
        import requests

        self.urls = [u.rstrip("/") for u in shard_urls]
        self.health = HealthTracker(len(self.urls), policy)
        self.timeout, self.probe_interval = request_timeout_s, probe_interval_s
        self.max_attempts = max_attempts or max(2, len(self.urls))
        self._http = session or requests.Session()
        self._inflight = [0] * len(self.urls)
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self._prober: Optional[threading.Thread] = None
        self.stats = dict(requests=0, retries=0, failures=0)

    # ------------------------------------------------------------------ shard choice
    def _pick(self, exclude: set[int]) -> int:
        cand = [i for i in self.health.select(include_suspect=True) if i not in exclude]
        if not cand:
            raise NoHealthyShardError(f"no serviceable generation shard ({self.health.summary()})")
        with self._lock:
            healthy = [i for i in cand if self.health.state(i) == ShardState.HEALTHY] or cand
            i = min(healthy, key=lambda j: self._inflight[j])
            self._inflight[i] += 1
        return i

    def post(self, path: str, body: dict) -> dict:
        """Forwards one JSON request; fails over to other shards on transport errors and 5xx answers."""
        self.stats["requests"] += 1
        tried: set[int] = set()
        last = ""
        for attempt in range(self.max_attempts):
            try:
                i = self._pick(tried)
            except NoHealthyShardError:
                if not tried:
                    raise
                break
            try:
                r = self._http.post(self.urls[i] + path, json=body, timeout=self.timeout)
                if r.status_code >= 500:
                    raise RuntimeError(f"HTTP {r.status_code}: {r.text[:200]}")
                self.health.report_success(i)
                out = r.json()
                if isinstance(out, dict):
                    out.setdefault("served_by", i)
                if r.status_code >= 400:
                    raise ValueError(out)   # the request itself is wrong: no retry elsewhere
                return out
            except ValueError:
                raise
            except Exception as e:
                last = f"{type(e).__name__}: {e}"
                self.health.report_failure(i, last)
                tried.add(i)
                if attempt + 1 < self.max_attempts:
                    self.stats["retries"] += 1
            finally:
                with self._lock:
                    self._inflight[i] -= 1
        self.stats["failures"] += 1
        raise NoHealthyShardError(f"request failed on shards {sorted(tried)}: {last}")

    def completions(self, **body) -> dict:
        return self.post("/v1/completions", body)

    def chat(self, **body) -> dict:
        return self.post("/v1/chat/completions", body)

    # ------------------------------------------------------------------ background probing of dead shards
    def probe_once(self) -> dict[int, bool]:
        """Asks every DEAD shard for ``/health``; one that answers goes through RESTARTING back to service."""
        out = {}
        for i, url in enumerate(self.urls):
            if self.health.state(i) != ShardState.DEAD:
                continue
            if self.health.begin_restart(i) != ShardState.RESTARTING:
                continue
            ok, version = False, None
            try:
                r = self._http.get(url + "/health", timeout=min(5.0, self.timeout))
                ok = r.status_code == 200
                version = (r.json() or {}).get("weight_version") if ok else None
            except Exception:
                ok = False
            self.health.finish_restart(i, ok, weight_version=version)
            out[i] = ok
        return out

    def start_probing(self) -> "GenerationRouter":
        def run():
            while not self._stop.wait(self.probe_interval):
                self.probe_once()

        self._prober = threading.Thread(target=run, daemon=True, name="rlb-router-probe")
        self._prober.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._prober is not None:
            self._prober.join(2.0)

    def set_weight_version(self, version: int, updated: Optional[list[int]] = None) -> None:
        self.health.set_weight_version(version, updated)


def create_router_app(router: GenerationRouter):
    """The router as a server of its own: same paths as a shard, plus ``/fleet`` with the health summary."""
    from fastapi import FastAPI, HTTPException

    app = FastAPI(title="rl_b200 generation router")

    def fwd(path: str, body: dict) -> Any:
        try:
            return router.post(path, body)
        except NoHealthyShardError as e:
            raise HTTPException(status_code=503, detail=str(e))
        except ValueError as e:
            raise HTTPException(status_code=400, detail=str(e))

    @app.post("/v1/completions")
    def completions(body: dict):
        return fwd("/v1/completions", body)

    @app.post("/v1/chat/completions")
    def chat(body: dict):
        return fwd("/v1/chat/completions", body)

    @app.post("/tokenize")
    def tokenize(body: dict):
        return fwd("/tokenize", body)

    @app.get("/fleet")
    def fleet():
        return dict(summary=router.health.summary(), serviceable=router.health.serviceable(), stats=router.stats,
                    shards=[dict(url=u, state=router.health.state(i).value) for i, u in enumerate(router.urls)])

    @app.get("/health")
    def health():
        if not router.health.serviceable():
            raise HTTPException(status_code=503, detail="fleet not serviceable")
        return {"status": "ok"}

    return app
