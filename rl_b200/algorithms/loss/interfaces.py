"""Loss-function contract (the role of nemo_rl/algorithms/loss/interfaces.py:23-110).

A loss function receives per-token quantities for one micro-batch plus the *global* count of valid sequences and
tokens of the whole optimizer step. Every metric it returns is already divided by that global count, so summing a
metric over micro-batches and data-parallel ranks yields the global mean.
"""

from __future__ import annotations

import enum
from typing import Any, Protocol

import torch


class LossType(enum.Enum):
    TOKEN_LEVEL = "token_level"
    SEQUENCE_LEVEL = "sequence_level"


class LossInputType(enum.Enum):
    LOGPROB = "logprob"            # next-token log-probabilities [B, S-1]
    LOGIT = "logit"                # full logits [B, S, V]
    DISTILLATION = "distillation"  # student top-k logits aligned with teacher top-k
    DRAFT = "draft"                # draft-model logits for speculative-decoding heads
    VALUE = "value"                # scalar value predictions [B, S]


class LossFunction(Protocol):
    loss_type: LossType
    input_type: LossInputType

    def __call__(self, data: Any, global_valid_seqs: torch.Tensor, global_valid_toks: torch.Tensor,
                 **loss_input: torch.Tensor) -> tuple[torch.Tensor, dict[str, Any]]: ...
