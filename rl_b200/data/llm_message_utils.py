"""Message-log <-> flat tensor conversions, loss masks and chat-template tokenisation
(the role of nemo_rl/data/llm_message_utils.py:59-846)."""

from __future__ import annotations

from typing import Any, Optional, Sequence

import torch

from rl_b200.distributed.batched_data_dict import BatchedDataDict

from .interfaces import LLMMessageLogType

TENSOR_KEYS_DEFAULT_PAD = {"token_ids": None, "generation_logprobs": 0.0, "token_loss_mask": 0}


def message_log_to_flat_messages(message_log: LLMMessageLogType) -> dict[str, Any]:
    """Concatenates every tensor key over the messages of one log; non-tensor keys become lists."""
    out: dict[str, Any] = {}
    keys = set().union(*[m.keys() for m in message_log]) if message_log else set()
    for k in keys:
        vals = [m[k] for m in message_log if k in m]
        if vals and all(isinstance(v, torch.Tensor) for v in vals):
            out[k] = torch.cat([v.reshape(-1) if v.dim() == 0 else v for v in vals]) if vals else torch.empty(0)
        else:
            out[k] = vals
    return out


def add_loss_mask_to_message_log(message_logs: Sequence[LLMMessageLogType], roles_to_train_on: Sequence[str] = ("assistant",),
                                 only_unmask_final: bool = False) -> None:
    """Adds ``token_loss_mask`` (1 on tokens of the trained roles) to every message in place."""
    for log in message_logs:
        last_trainable = max((i for i, m in enumerate(log) if m["role"] in roles_to_train_on), default=-1)
        for i, m in enumerate(log):
            on = m["role"] in roles_to_train_on and (not only_unmask_final or i == last_trainable)
            m["token_loss_mask"] = torch.ones_like(m["token_ids"]) if on else torch.zeros_like(m["token_ids"])


def get_keys_from_message_log(message_log: LLMMessageLogType, keys: Sequence[str]) -> LLMMessageLogType:
    return [{k: m[k] for k in keys if k in m} for m in message_log]


def batched_message_log_to_flat_message(message_logs: Sequence[LLMMessageLogType], pad_value_dict: Optional[dict] = None,
                                        make_sequence_length_divisible_by: int = 1):
    """List of message logs -> (BatchedDataDict of right-padded [B, S] tensors per tensor key, input_lengths [B])."""
    pad_value_dict = pad_value_dict or {}
    flats = [message_log_to_flat_messages(ml) for ml in message_logs]
    lengths = torch.tensor([int(f["token_ids"].numel()) if "token_ids" in f else 0 for f in flats], dtype=torch.long)
    S = int(lengths.max()) if len(flats) else 0
    m = make_sequence_length_divisible_by
    if m > 1:
        S = -(-S // m) * m
    out = BatchedDataDict()
    tensor_keys = set()
    for f in flats:
        tensor_keys |= {k for k, v in f.items() if isinstance(v, torch.Tensor)}
    for k in tensor_keys:
        proto = next(f[k] for f in flats if k in f)
        if proto.dim() >= 2:   # per-sample rows of another modality (image patches): kept ragged, one entry per sample
            from .multimodal_utils import PackedTensor

            out[k] = PackedTensor([f.get(k) for f in flats])
            continue
        pad = pad_value_dict.get(k, 0)
        buf = torch.full((len(flats), S), pad, dtype=proto.dtype)
        for i, f in enumerate(flats):
            if k in f:
                v = f[k]
                buf[i, : v.numel()] = v
        out[k] = buf
    for k in set().union(*[f.keys() for f in flats]) - tensor_keys if flats else ():
        out[k] = [f.get(k) for f in flats]
    if "image_sizes" in out:   # per message lists of patch counts -> one list per sample
        out["image_sizes"] = [[int(s) for per_msg in (row or []) for s in per_msg] for row in out["image_sizes"]]
    return out, lengths


MULTIMODAL_KEYS = ("pixel_patches", "image_sizes")


def multimodal_fields(flat: BatchedDataDict) -> dict[str, Any]:
    """The image fields of a flattened batch (empty for text-only data), to be carried into train / generation batches."""
    return {k: flat[k] for k in MULTIMODAL_KEYS if k in flat}


def get_formatted_message_log(message_log: list[dict[str, str]], tokenizer, task_data_spec=None,
                              add_bos_token: bool = True, add_eos_token: bool = True,
                              add_generation_prompt: bool = False) -> LLMMessageLogType:
    """Tokenises a chat with the tokenizer's template message by message, so that every message owns exactly the
    tokens the template emits for it (prefix-difference method)."""
    out: LLMMessageLogType = []
    prev = ""
    for i, msg in enumerate(message_log):
        is_last = i == len(message_log) - 1
        text = tokenizer.apply_chat_template(message_log[: i + 1], tokenize=False,
                                             add_generation_prompt=add_generation_prompt and is_last)
        piece = text[len(prev):] if text.startswith(prev) else text
        prev = text
        if i == 0 and not add_bos_token and tokenizer.bos_token and piece.startswith(tokenizer.bos_token):
            piece = piece[len(tokenizer.bos_token):]
        if is_last and add_eos_token and tokenizer.eos_token and not add_generation_prompt and not piece.rstrip("\n").endswith(tokenizer.eos_token):
            piece = piece + tokenizer.eos_token
        ids = tokenizer(piece, add_special_tokens=False, return_tensors="pt")["input_ids"][0]
        new = dict(msg)
        new["token_ids"] = ids
        new["content"] = piece
        out.append(new)
    return out
