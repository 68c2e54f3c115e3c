"""Environment for single-turn vision-language tasks: reward 1 when the response names the ground-truth label (exact
word match, case-insensitive; an optional ``\\boxed{}`` / ``<answer>`` wrapper is unwrapped first), plus an optional small
format reward. Role of nemo_rl/environments/vlm_environment.py."""

from __future__ import annotations

import re
from typing import Optional

import torch

from .interfaces import EnvironmentReturn


def extract_answer(text: str) -> str:
    for pat in (r"<answer>(.*?)</answer>", r"\\boxed\{([^}]*)\}"):
        m = re.search(pat, text, flags=re.S)
        if m:
            return m.group(1).strip()
    return text.strip()


class VLMEnvironment:
    def __init__(self, cfg: Optional[dict] = None):
        c = dict(format_reward=0.0, exact=False)
        c.update(cfg or {})
        self.cfg = c

    def step(self, message_log_batch, metadata) -> EnvironmentReturn:
        rewards, answers = [], []
        for log, meta in zip(message_log_batch, metadata):
            resp = next((m["content"] for m in reversed(log) if m["role"] == "assistant"), "")
            ans = extract_answer(resp)
            gt = str((meta or {}).get("ground_truth", "")).strip().lower()
            if self.cfg["exact"]:
                ok = ans.lower() == gt
            else:
                ok = bool(gt) and re.search(r"(?<![a-z0-9])" + re.escape(gt) + r"(?![a-z0-9])", ans.lower()) is not None
            fmt = self.cfg["format_reward"] if ("<answer>" in resp or "\\boxed{" in resp) else 0.0
            rewards.append(float(ok) + fmt)
            answers.append(ans)
        n = len(message_log_batch)
        return EnvironmentReturn(observations=[{"role": "environment", "content": ""} for _ in range(n)], metadata=list(metadata),
                                 next_stop_strings=[None] * n, rewards=torch.tensor(rewards, dtype=torch.float32),
                                 terminateds=torch.ones(n, dtype=torch.bool), answers=answers)

    def global_post_process_and_metrics(self, batch):
        r = batch["total_reward"] if "total_reward" in batch else batch["rewards"]
        return batch, {"accuracy": float((r >= 1.0).float().mean()) if len(r) else 0.0}

    def shutdown(self) -> None:
        pass
