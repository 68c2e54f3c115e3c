"""From a finished prompt group to rows in the data plane.

``record_to_train_batch`` flattens the completions of one prompt (message logs with token ids, log-probabilities and a reward
each) into the padded training batch the loss consumes; ``pack_payload`` turns such a batch into what a data-plane ``put``
needs: one key, one record (variable-length fields cut to the sample's length) and one :class:`SampleMeta` per row, stamped
with the weight version that produced the samples. Role of nemo_rl/experience/payload.py:31-128.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Sequence

import torch

from rl_b200.data.llm_message_utils import batched_message_log_to_flat_message
from rl_b200.data_plane import SampleMeta
from rl_b200.data_plane.codec import batch_to_records
from rl_b200.distributed.batched_data_dict import BatchedDataDict

TOKEN_ALIGNED_FIELDS = ("input_ids", "token_mask", "generation_logprobs", "prev_logprobs", "reference_policy_logprobs", "advantages",
                        "routed_experts")


@dataclass
class Completion:
    message_log: list            # the whole conversation: prompt messages followed by generated / environment turns
    reward: float = 0.0
    truncated: bool = False


@dataclass
class PromptGroupRecord:
    """All completions sampled for one prompt."""

    prompt: list                 # the prompt's messages (with ``token_ids``)
    completions: list[Completion] = field(default_factory=list)
    prompt_idx: int = 0


def record_to_train_batch(record: PromptGroupRecord, pad_value_dict: Optional[Mapping[str, int]] = None) -> BatchedDataDict:
    """N completions -> N rows: ``input_ids``, ``input_lengths``, ``token_mask`` (1 on generated tokens), ``sample_mask``,
    ``generation_logprobs``, ``prompt_ids_for_adv`` (the prompt alone, the grouping key of the advantage estimator),
    ``total_reward``."""
    from rl_b200.algorithms.grpo import build_train_data

    n = len(record.completions)
    assert n > 0, "PromptGroupRecord has no completions"
    pad = dict(pad_value_dict or {"token_ids": 0})
    logs = [[dict(m) for m in c.message_log] for c in record.completions]
    batch = BatchedDataDict({"message_log": logs, "loss_multiplier": torch.ones(n)})
    td = build_train_data(batch, pad.get("token_ids", 0))
    prompt_flat, _ = batched_message_log_to_flat_message([[dict(m) for m in record.prompt] for _ in range(n)], pad)
    td["prompt_ids_for_adv"] = prompt_flat["token_ids"]
    td["total_reward"] = torch.tensor([float(c.reward) for c in record.completions], dtype=torch.float32)
    td["truncated"] = torch.tensor([float(c.truncated) for c in record.completions], dtype=torch.float32)
    return td


def pack_payload(train_batch: Mapping[str, Any], weight_version: int, group_id: str,
                 token_aligned_fields: Sequence[str] = TOKEN_ALIGNED_FIELDS) -> tuple[list[str], list[dict], list[SampleMeta]]:
    """(keys ``{group_id}_g{i}``, per-row records with the token-aligned fields cut to the row's length, per-row metadata
    carrying the weight version and the group). The caller owns the uniqueness of ``group_id``."""
    batch = train_batch if isinstance(train_batch, BatchedDataDict) else BatchedDataDict(dict(train_batch))
    jag = [f for f in token_aligned_fields if f in batch]
    recs = batch_to_records(batch, jagged=jag)
    keys = [f"{group_id}_g{i}" for i in range(len(recs))]
    metas = [SampleMeta(k, num_tokens=int(r["input_lengths"]), weight_version=int(weight_version), group=str(group_id)) for k, r in zip(keys, recs)]
    return keys, recs, metas
