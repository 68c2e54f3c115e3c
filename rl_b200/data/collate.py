"""Collate functions (nemo_rl/data/collate_fn.py:29-150): lists of DatumSpec -> BatchedDataDict."""

from __future__ import annotations

from typing import Any, Sequence

import torch

from rl_b200.distributed.batched_data_dict import BatchedDataDict

from .llm_message_utils import add_loss_mask_to_message_log, batched_message_log_to_flat_message, multimodal_fields


def rl_collate_fn(batch: Sequence[dict]) -> BatchedDataDict:
    """Keeps message logs as python lists (rollouts extend them) and stacks the scalars."""
    out = BatchedDataDict(
        message_log=[d["message_log"] for d in batch],
        length=torch.tensor([d["length"] for d in batch], dtype=torch.long),
        loss_multiplier=torch.tensor([float(d.get("loss_multiplier", 1.0)) for d in batch]),
        extra_env_info=[d.get("extra_env_info") for d in batch],
        task_name=[d.get("task_name", "default") for d in batch],
        idx=torch.tensor([int(d.get("idx", i)) for i, d in enumerate(batch)], dtype=torch.long),
        batch_max_length=torch.full((len(batch),), max((d["length"] for d in batch), default=0), dtype=torch.long),
    )
    ss = [d.get("stop_strings") for d in batch]
    if any(s is not None for s in ss):
        out["stop_strings"] = ss
    return out


def eval_collate_fn(batch: Sequence[dict]) -> BatchedDataDict:
    return rl_collate_fn(batch)


def sft_collate_fn(batch: Sequence[dict], pad_token_id: int = 0, make_sequence_length_divisible_by: int = 1,
                   roles_to_train_on=("assistant",), only_unmask_final: bool = False) -> BatchedDataDict:
    """Flat [B, S] token batch with ``token_mask`` on the trained roles and ``sample_mask`` from loss multipliers."""
    logs = [d["message_log"] for d in batch]
    add_loss_mask_to_message_log(logs, roles_to_train_on, only_unmask_final)
    flat, lengths = batched_message_log_to_flat_message(logs, {"token_ids": pad_token_id}, make_sequence_length_divisible_by)
    return BatchedDataDict(
        input_ids=flat["token_ids"], input_lengths=lengths, token_mask=flat["token_loss_mask"].float(),
        sample_mask=torch.tensor([float(d.get("loss_multiplier", 1.0)) for d in batch]), **multimodal_fields(flat),
    )


def preference_collate_fn(batch: Sequence[dict], pad_token_id: int = 0, make_sequence_length_divisible_by: int = 1) -> BatchedDataDict:
    """Interleaves chosen / rejected rows: row 2i is the chosen response of pair i, row 2i+1 its rejected one."""
    logs, mults = [], []
    for d in batch:
        logs += [d["message_log_chosen"], d["message_log_rejected"]]
        mults += [float(d.get("loss_multiplier", 1.0))] * 2
    add_loss_mask_to_message_log(logs, ("assistant",), only_unmask_final=True)
    flat, lengths = batched_message_log_to_flat_message(logs, {"token_ids": pad_token_id}, make_sequence_length_divisible_by)
    return BatchedDataDict(input_ids=flat["token_ids"], input_lengths=lengths, token_mask=flat["token_loss_mask"].float(),
                           sample_mask=torch.tensor(mults))
