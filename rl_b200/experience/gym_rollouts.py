"""Rollouts owned by a gym: the agent server runs the whole episode (turns, tools, verification) and calls the policy
through its OpenAI-compatible endpoint (``rl_b200/engine/http_server.py``); the trainer posts one row per sample, gets
back the reward and the episode's messages with the token ids and log-probabilities the policy server reported, and turns
them into the message logs the losses consume.

Rows complete in arbitrary order; prompt groups (``num_generations`` consecutive rows) are yielded as soon as their last
row is back, with the rows restored to input order inside the group, so training can start on early groups while slow
episodes are still running. A row whose transport keeps failing is an infrastructure failure (retried, then raised); a
row whose result cannot be used (token ids that do not extend the previous turn, missing log-probabilities) is a data
failure: the sample is kept with ``loss_multiplier`` 0. Optional penalties: malformed tool-call markers left in an
assistant turn, unbalanced thinking tags.

Role of ``run_async_nemo_gym_rollout`` / ``run_nemo_gym_rollout_sync`` and the NeMo-Gym environment actor
(nemo_rl/experience/rollouts.py:1585, :2261, :2505; nemo_rl/environments/nemo_gym.py).
"""

from __future__ import annotations

import concurrent.futures as cf
from dataclasses import dataclass, field
from typing import Any, Callable, Iterator, Optional, Sequence

import torch

from rl_b200.distributed.batched_data_dict import BatchedDataDict
from rl_b200.experience.failures import DataFailure, InfraFailure

DEFAULT_INVALID_TOOL_CALL_PATTERNS = ("<tool_call>", "</tool_call>", "<function_call>", "</function_call>")
DEFAULT_THINKING_TAGS = ("<think>", "</think>")


class GymClient:
    """POSTs rows to an agent server's ``/run`` endpoint. The body carries the row, the base URL of the policy server the
    agent must call and the sampling parameters; the reply carries ``reward`` and ``response.output`` (the episode)."""

    def __init__(self, url: str, policy_base_url: str, timeout_s: float = 1800.0, max_retries: int = 2, post: Optional[Callable] = None):
        self.url, self.policy_base_url = url.rstrip("/"), policy_base_url
        self.timeout_s, self.max_retries = timeout_s, max_retries
        self._post = post
        self._session = None

    def run(self, row: dict, sampling: Optional[dict] = None) -> dict:
        body = dict(row=row, policy_base_url=self.policy_base_url, sampling=dict(sampling or {}))
        last: Optional[Exception] = None
        for _ in range(self.max_retries + 1):
            try:
                if self._post is not None:
                    return self._post(self.url + "/run", body, self.timeout_s)
                if self._session is None:
                    import requests

                    self._session = requests.Session()
                r = self._session.post(self.url + "/run", json=body, timeout=self.timeout_s)
                if r.status_code >= 500 or r.status_code in (408, 429):
                    raise ConnectionError(f"HTTP {r.status_code}: {r.text[:200]}")
                if r.status_code >= 400:   # the server understood and refused: retrying will not help
                    raise DataFailure(f"gym refused the row: HTTP {r.status_code}: {r.text[:200]}")
                return r.json()
            except DataFailure:
                raise
            except Exception as e:
                last = e
        raise InfraFailure(f"gym server {self.url} failed after {self.max_retries + 1} attempts: {last}")


@dataclass
class GymRolloutResult:
    """One finished prompt group."""

    group_index: int
    rows: list[int]                          # input indices of the group's rows, ascending
    message_logs: list[list[dict]]
    rewards: torch.Tensor                    # [n] after penalties
    raw_rewards: torch.Tensor
    loss_multiplier: torch.Tensor            # 0 for rows that must not train (data failures, samples the gym flagged)
    truncated: torch.Tensor
    metrics: dict = field(default_factory=dict)


def _text_of(item: dict) -> str:
    c = item.get("content", "")
    if isinstance(c, list):
        return "".join(str(p.get("text", "")) for p in c if isinstance(p, dict))
    return str(c)


def episode_to_message_log(output: Sequence[dict], tokenizer=None) -> tuple[list[dict], int]:
    """The gym's ``response.output`` -> message log. Assistant items carry ``prompt_token_ids`` (everything the policy saw),
    ``generation_token_ids`` and ``generation_log_probs``; whatever the prompt of turn i + 1 adds beyond turn i's prompt +
    generation is the environment's / tool's contribution and becomes a non-trainable message. Returns the log and the number
    of generated tokens. Raises :class:`DataFailure` when a turn's prompt does not extend the tokens seen so far."""
    log: list[dict] = []
    seen: list[int] = []
    gen_tokens = 0
    for item in output:
        role = item.get("role", "assistant" if "generation_token_ids" in item else "environment")
        if "generation_token_ids" not in item:
            continue   # tool / environment text arrives through the next assistant turn's prompt tokens
        p, g, lp = list(item.get("prompt_token_ids") or []), list(item["generation_token_ids"]), item.get("generation_log_probs")
        if lp is None or len(lp) != len(g):
            raise DataFailure("an assistant turn came back without one log-probability per generated token")
        if p[: len(seen)] != seen:
            raise DataFailure("a turn's prompt tokens do not extend the previous turn (re-tokenisation changed the history)")
        new = p[len(seen):]
        if new:
            log.append({"role": "user" if not log else "environment", "content": tokenizer.decode(new) if tokenizer is not None else "",
                        "token_ids": torch.tensor(new, dtype=torch.long)})
        log.append({"role": role, "content": _text_of(item) or (tokenizer.decode(g) if tokenizer is not None else ""),
                    "token_ids": torch.tensor(g, dtype=torch.long), "generation_logprobs": torch.tensor(lp, dtype=torch.float32)})
        seen = p + g
        gen_tokens += len(g)
    if not gen_tokens:
        raise DataFailure("the episode holds no generated tokens")
    return log, gen_tokens


def reward_penalty(log: Sequence[dict], cfg: Optional[dict]) -> float:
    """Penalty to subtract: ``invalid_tool_call_penalty`` when an assistant turn still contains raw tool-call markers (the
    server failed to parse them), ``thinking_penalty`` when thinking tags are unbalanced."""
    if not cfg:
        return 0.0
    pen = 0.0
    pats = tuple(cfg.get("invalid_tool_call_patterns") or DEFAULT_INVALID_TOOL_CALL_PATTERNS)
    open_t, close_t = tuple(cfg.get("thinking_tags") or DEFAULT_THINKING_TAGS)
    for m in log:
        if m["role"] != "assistant":
            continue
        text = str(m.get("content", ""))
        if cfg.get("invalid_tool_call_penalty") and any(p in text for p in pats):
            pen += float(cfg["invalid_tool_call_penalty"])
        if cfg.get("thinking_penalty") and text.count(open_t) != text.count(close_t):
            pen += float(cfg["thinking_penalty"])
    return pen


def run_gym_rollout(rows: Sequence[dict], client, tokenizer=None, num_generations: int = 1, sampling: Optional[dict] = None,
                    max_workers: int = 64, reward_penalty_config: Optional[dict] = None, mask_env_flagged_samples: bool = True,
                    max_seq_len: Optional[int] = None) -> Iterator[GymRolloutResult]:
    """Streams finished prompt groups in completion order. ``rows``: one dict per sample (``num_generations`` consecutive
    rows form a group); ``client.run(row, sampling)`` performs the episode."""
    n = len(rows)
    assert n % num_generations == 0, "rows must come in whole prompt groups"
    done: dict[int, tuple] = {}
    pending = {g: num_generations for g in range(n // num_generations)}
    with cf.ThreadPoolExecutor(max_workers=max(1, min(max_workers, n))) as ex:
        futs = {ex.submit(client.run, rows[i], sampling): i for i in range(n)}
        for fut in cf.as_completed(futs):
            i = futs[fut]
            try:
                res = fut.result()
                log, gen = episode_to_message_log((res.get("response") or {}).get("output") or [], tokenizer)
                raw = float(res.get("reward", 0.0))
                length = sum(int(m["token_ids"].numel()) for m in log)
                trunc = bool(res.get("truncated", False)) or (max_seq_len is not None and length >= max_seq_len)
                mult = 0.0 if (mask_env_flagged_samples and res.get("mask_sample")) else 1.0
                done[i] = (log, raw, raw - reward_penalty(log, reward_penalty_config), mult, trunc, gen, None)
            except DataFailure as e:      # unusable result: keep the row (group statistics need it), do not train on it
                stub = [{"role": "user", "content": "", "token_ids": torch.zeros(1, dtype=torch.long)},
                        {"role": "assistant", "content": "", "token_ids": torch.zeros(1, dtype=torch.long),
                         "generation_logprobs": torch.zeros(1)}]
                done[i] = (stub, 0.0, 0.0, 0.0, False, 0, str(e))
            g = i // num_generations
            pending[g] -= 1
            if pending[g] == 0:
                idx = list(range(g * num_generations, (g + 1) * num_generations))
                parts = [done.pop(j) for j in idx]
                yield GymRolloutResult(
                    group_index=g, rows=idx, message_logs=[p[0] for p in parts],
                    raw_rewards=torch.tensor([p[1] for p in parts]), rewards=torch.tensor([p[2] for p in parts]),
                    loss_multiplier=torch.tensor([p[3] for p in parts]), truncated=torch.tensor([p[4] for p in parts]),
                    metrics=dict(generated_tokens=float(sum(p[5] for p in parts)), data_failures=float(sum(p[6] is not None for p in parts)),
                                 mean_reward=float(sum(p[2] for p in parts)) / len(parts)))


def run_gym_rollout_sync(batch: BatchedDataDict, client, tokenizer=None, num_generations: int = 1, **kw) -> tuple[BatchedDataDict, dict]:
    """The whole batch at once, rows back in input order: ``batch['extra_env_info']`` holds the gym rows. Returns the batch
    with ``message_log``, ``total_reward``, ``loss_multiplier``, ``truncated`` and rollout metrics."""
    rows = list(batch["extra_env_info"])
    n = len(rows)
    logs: list = [None] * n
    rewards, mult, trunc = torch.zeros(n), torch.ones(n), torch.zeros(n, dtype=torch.bool)
    metrics = dict(generated_tokens=0.0, data_failures=0.0, groups=0.0)
    order = []
    for res in run_gym_rollout(rows, client, tokenizer, num_generations, **kw):
        order.append(res.group_index)
        for k, i in enumerate(res.rows):
            logs[i] = res.message_logs[k]
            rewards[i], mult[i], trunc[i] = res.rewards[k], res.loss_multiplier[k], res.truncated[k]
        metrics["generated_tokens"] += res.metrics["generated_tokens"]
        metrics["data_failures"] += res.metrics["data_failures"]
        metrics["groups"] += 1
    out = BatchedDataDict(dict(batch))
    out["message_log"] = logs
    out["total_reward"] = rewards
    base = batch["loss_multiplier"].float() if "loss_multiplier" in batch else torch.ones(n)
    out["loss_multiplier"] = base * mult
    out["truncated"] = trunc
    metrics["mean_reward"] = float(rewards.mean()) if n else 0.0
    metrics["group_completion_order"] = order
    return out, metrics
