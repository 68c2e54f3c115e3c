"""Environments behind HTTP: a resource server owns the task logic (verifiers, tools, simulators) and the trainer talks
to it with the ordinary environment contract. ``RemoteEnvironment`` is the client side (``step`` posts the message logs
and metadata, gets rewards / observations / termination flags back); ``create_env_app`` wraps any local environment as
such a server. This is the integration style of the reference's NeMo-Gym environment (nemo_rl/environments/nemo_gym.py):
the agent / resource servers live in their own processes and may themselves call the policy through the generation
HTTP front end (``rl_b200/engine/http_server.py``).
"""

from __future__ import annotations

from typing import Any, Optional

import torch

from .interfaces import EnvironmentReturn


def _plain_log(log: list[dict]) -> list[dict]:
    """Message logs carry token tensors; the wire format keeps roles and text (and token ids as lists when asked)."""
    return [{k: (v.tolist() if isinstance(v, torch.Tensor) else v) for k, v in m.items() if k in ("role", "content", "token_ids")} for m in log]


class RemoteEnvironment:
    def __init__(self, cfg: Optional[dict] = None):
        c = dict(url=None, timeout_s=300.0, max_retries=2, send_token_ids=False, batch_size=256)
        c.update(cfg or {})
        assert c["url"], "remote environment needs cfg.url"
        self.cfg = c
        import requests

        self._http = requests.Session()

    def _post(self, path: str, body: dict) -> dict:
        last: Optional[Exception] = None
        for _ in range(int(self.cfg["max_retries"]) + 1):
            try:
                r = self._http.post(self.cfg["url"].rstrip("/") + path, json=body, timeout=self.cfg["timeout_s"])
                if r.status_code >= 500:
                    raise RuntimeError(f"HTTP {r.status_code}: {r.text[:200]}")
                r.raise_for_status()
                return r.json()
            except Exception as e:   # the rollout layer decides what a lost environment means for the sample
                last = e
        raise ConnectionError(f"environment server {self.cfg['url']} failed: {last}")

    def step(self, message_log_batch, metadata) -> EnvironmentReturn:
        n, bs = len(message_log_batch), int(self.cfg["batch_size"])
        obs, meta, stops, rewards, term, answers = [], [], [], [], [], []
        for s in range(0, n, bs):
            logs = [_plain_log(l) for l in message_log_batch[s : s + bs]]
            if not self.cfg["send_token_ids"]:
                for l in logs:
                    for m in l:
                        m.pop("token_ids", None)
            out = self._post("/step", {"message_logs": logs, "metadata": list(metadata[s : s + bs])})
            k = len(logs)
            obs += out.get("observations") or [{"role": "environment", "content": ""}] * k
            meta += out.get("metadata") or list(metadata[s : s + bs])
            stops += out.get("next_stop_strings") or [None] * k
            rewards += out["rewards"]
            term += out.get("terminateds") or [True] * k
            answers += out.get("answers") or [None] * k
        return EnvironmentReturn(observations=obs, metadata=meta, next_stop_strings=stops, rewards=torch.tensor(rewards, dtype=torch.float32),
                                 terminateds=torch.tensor(term, dtype=torch.bool), answers=answers)

    def global_post_process_and_metrics(self, batch):
        r = batch["total_reward"] if "total_reward" in batch else batch["rewards"]
        return batch, {"mean_reward": float(r.float().mean()) if len(r) else 0.0}

    def shutdown(self) -> None:
        self._http.close()


def create_env_app(env: Any):
    """Serves a local environment object over HTTP (``POST /step``, ``GET /health``)."""
    from fastapi import FastAPI

    app = FastAPI(title="rl_b200 environment server")

    @app.get("/health")
    def health():
        return {"status": "ok", "environment": type(env).__name__}

    @app.post("/step")
    def step(body: dict):
        r = env.step(body["message_logs"], body.get("metadata") or [None] * len(body["message_logs"]))
        rew = r.rewards
        return dict(observations=r.observations, metadata=r.metadata, next_stop_strings=r.next_stop_strings,
                    rewards=rew.tolist() if isinstance(rew, torch.Tensor) else list(rew),
                    terminateds=r.terminateds.tolist() if isinstance(r.terminateds, torch.Tensor) else list(r.terminateds), answers=r.answers)

    return app
