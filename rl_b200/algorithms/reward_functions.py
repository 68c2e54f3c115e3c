"""Reward shaping applied after the environments score a batch (nemo_rl/algorithms/reward_functions.py:24-171).

* DAPO over-long shaping: responses longer than ``max_response_length - overlong_buffer_length`` lose reward linearly,
  ``-overlong_buffer_penalty`` at ``max_response_length`` and more beyond it.
* Stop-properly penalty: truncated responses are scaled by ``stop_properly_penalty_coef`` (0 zeroes them, 1 keeps).
"""

from __future__ import annotations

from typing import Optional

import torch

REWARD_SHAPING_DEFAULTS = dict(enabled=False, overlong_buffer_length=None, overlong_buffer_penalty=None,
                               max_response_length=None, stop_properly_penalty_coef=None)


def apply_reward_shaping(batch, cfg: Optional[dict]):
    """Shapes ``batch['total_reward']`` in place (keeps the raw values in ``unshaped_reward``)."""
    c = dict(REWARD_SHAPING_DEFAULTS)
    c.update(cfg or {})
    if not c["enabled"]:
        return batch
    rewards = batch["total_reward"].clone().float()
    batch["unshaped_reward"] = batch["total_reward"].clone()
    gen_len = batch["response_token_lengths"] if "response_token_lengths" in batch else batch["generation_lengths"]
    gen_len = torch.as_tensor(gen_len).float()
    coef = c["stop_properly_penalty_coef"]
    if coef is not None:
        assert 0.0 <= coef <= 1.0, "stop_properly_penalty_coef must lie in [0, 1]"
        trunc = batch["truncated"].bool()
        rewards = torch.where(trunc, rewards * coef, rewards)
    else:
        L, buf, pen = c["max_response_length"], c["overlong_buffer_length"], c["overlong_buffer_penalty"]
        if L is None or buf is None or pen is None:
            raise ValueError("overlong shaping needs max_response_length, overlong_buffer_length and overlong_buffer_penalty")
        assert 0 < buf <= L, "overlong_buffer_length must lie in (0, max_response_length]"
        expected = L - buf
        excess = (gen_len - expected).clamp(min=0)
        rewards = rewards - excess / buf * pen   # no cap beyond max_response_length: the penalty keeps growing
    batch["total_reward"] = rewards
    return batch


REWARD_SCALING_DEFAULTS = dict(enabled=False, source_min=0.0, source_max=1.0, target_min=0.0, target_max=1.0)


def scale_rewards(batch, cfg: Optional[dict]):
    """Linear map of rewards from [source_min, source_max] (clamped) to [target_min, target_max]."""
    c = dict(REWARD_SCALING_DEFAULTS)
    c.update(cfg or {})
    if not c["enabled"]:
        return batch
    r = batch["total_reward"].float()
    lo, hi = c["source_min"], c["source_max"]
    r = r.clamp(lo, hi)
    batch["total_reward"] = c["target_min"] + (r - lo) / (hi - lo) * (c["target_max"] - c["target_min"])
    return batch
