"""Data contracts between datasets, environments and algorithms (nemo_rl/data/interfaces.py:24-117).

A *message log* is a list of messages ``{"role", "content", "token_ids" (1-D LongTensor), ...}``; tensor-valued extras
(``generation_logprobs``, ``token_loss_mask``) ride along per message and are concatenated when the log is flattened.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Optional, TypedDict

import torch

LLMMessageLogType = list[dict[str, Any]]


class DatumSpec(TypedDict, total=False):
    message_log: LLMMessageLogType
    length: int                    # total tokens in message_log
    extra_env_info: Optional[dict]  # whatever the environment needs to score the sample (ground truth, seeds...)
    loss_multiplier: float         # 0 masks the sample out of the loss (e.g. over-long prompts)
    idx: int
    task_name: str
    stop_strings: Optional[list[str]]


@dataclass
class TaskDataSpec:
    task_name: Optional[str] = None
    prompt_file: Optional[str] = None
    system_prompt_file: Optional[str] = None
    prompt: Optional[str] = None
    system_prompt: Optional[str] = None

    def __post_init__(self):
        def read(p):
            if p is None:
                return None
            with open(p) as f:
                return f.read()

        if self.prompt is None:
            self.prompt = read(self.prompt_file)
        if self.system_prompt is None:
            self.system_prompt = read(self.system_prompt_file)


TaskDataProcessFnCallable = Callable[[dict, TaskDataSpec, Any, int, int], DatumSpec]
