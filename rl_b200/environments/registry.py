"""Environment registry: ``env_name`` in the data config -> environment class."""

from __future__ import annotations

import importlib
from typing import Callable, Optional

_REGISTRY: dict[str, str] = {
    "math": "rl_b200.environments.math_environment:MathEnvironment",
    "math_default": "rl_b200.environments.math_environment:MathEnvironment",
    "token_fraction": "rl_b200.environments.synthetic:TokenFractionEnv",
    "hash_parity": "rl_b200.environments.synthetic:HashParityEnv",
    "sliding_puzzle": "rl_b200.environments.games.sliding_puzzle:SlidingPuzzleEnv",
    "code": "rl_b200.environments.code_environment:CodeEnvironment",
    "code_jaccard": "rl_b200.environments.code_environment:CodeJaccardEnvironment",
    "reward_model": "rl_b200.environments.reward_model_environment:RewardModelEnvironment",
    "dapo": "rl_b200.environments.math_environment:MathEnvironment",
    "math_multi_reward": "rl_b200.environments.math_environment:MathMultiRewardEnvironment",
    "multichoice": "rl_b200.environments.math_environment:MathEnvironment",
    "vlm": "rl_b200.environments.vlm_environment:VLMEnvironment",
    "tool": "rl_b200.environments.tool_environment:ToolEnvironment",
    "retriever": "rl_b200.environments.tool_environment:ToolEnvironment",
    "remote": "rl_b200.environments.remote_environment:RemoteEnvironment",
    "nemo_gym": "rl_b200.environments.remote_environment:RemoteEnvironment",
}


def register_env(name: str, target: str) -> None:
    _REGISTRY[name] = target


def create_env(name: str, cfg: Optional[dict] = None):
    if name not in _REGISTRY:
        raise KeyError(f"unknown environment '{name}' ({sorted(_REGISTRY)})")
    mod, cls = _REGISTRY[name].split(":")
    return getattr(importlib.import_module(mod), cls)(cfg or {})
