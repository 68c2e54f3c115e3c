"""Token-level synthetic environments for benchmarks and oracles: rewards computed from generated token ids, no
tokenizer or dataset required.

``TokenFractionEnv``  reward = fraction of generated tokens equal to a target id (the CPU/gloo oracle task).
``HashParityEnv``     reward = mean over generated tokens of the parity of a 32-bit integer hash of (token id, position),
                      a deterministic, cheap, unlearnable-by-accident signal with mean 0.5 for random text.
"""

from __future__ import annotations

from typing import Optional

import torch

from .interfaces import EnvironmentReturn


def _last_assistant_tokens(log: list[dict]) -> torch.Tensor:
    for m in reversed(log):
        if m["role"] == "assistant":
            return m["token_ids"]
    return torch.empty(0, dtype=torch.long)


class _TokenEnvBase:
    def _score(self, toks: torch.Tensor) -> float:
        raise NotImplementedError

    def step(self, message_log_batch, metadata) -> EnvironmentReturn:
        rewards = torch.tensor([self._score(_last_assistant_tokens(log)) for log in message_log_batch], dtype=torch.float32)
        n = len(message_log_batch)
        return EnvironmentReturn(
            observations=[{"role": "environment", "content": ""} for _ in range(n)],
            metadata=list(metadata), next_stop_strings=[None] * n, rewards=rewards,
            terminateds=torch.ones(n, dtype=torch.bool), answers=[None] * n)

    def global_post_process_and_metrics(self, batch):
        r = batch["total_reward"] if "total_reward" in batch else batch.get("rewards")
        return batch, {"mean_reward": float(r.float().mean()) if r is not None and len(r) else 0.0}

    def shutdown(self):
        pass


class TokenFractionEnv(_TokenEnvBase):
    def __init__(self, cfg: Optional[dict] = None):
        self.target = int((cfg or {}).get("target_token_id", 7))

    def _score(self, toks):
        return float((toks == self.target).float().mean()) if toks.numel() else 0.0


class HashParityEnv(_TokenEnvBase):
    def __init__(self, cfg: Optional[dict] = None):
        self.salt = int((cfg or {}).get("salt", 0x9E3779B1))

    def _score(self, toks):
        if not toks.numel():
            return 0.0
        x = toks.to(torch.int64) * 2654435761 + torch.arange(toks.numel(), dtype=torch.int64) * self.salt
        x = (x ^ (x >> 15)) & 0xFFFFFFFF
        x = (x * 2246822519) & 0xFFFFFFFF
        x = x ^ (x >> 13)
        return float((x & 1).float().mean())
