"""Environment contract (nemo_rl/environments/interfaces.py:26-90)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional, Protocol

import torch


@dataclass
class EnvironmentReturn:
    observations: list[dict[str, str]]      # one message per sample appended to the log (role "environment"/"user")
    metadata: list[Optional[dict]]          # updated extra_env_info per sample
    next_stop_strings: list[Optional[list[str]]]
    rewards: torch.Tensor                   # [B] (or [B, K] for multi-component rewards)
    terminateds: torch.Tensor               # [B] bool: episode over
    answers: Optional[list[Optional[str]]] = None


class EnvironmentInterface(Protocol):
    def step(self, message_log_batch: list[list[dict]], metadata: list[Optional[dict]]) -> EnvironmentReturn: ...

    def global_post_process_and_metrics(self, batch) -> tuple[Any, dict]: ...

    def shutdown(self) -> None: ...
