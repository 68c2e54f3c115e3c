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


def get_first_index_that_differs(a: str, b: str) -> int:
    """Length of the common prefix of two strings."""
    n = min(len(a), len(b))
    for i in range(n):
        if a[i] != b[i]:
            return i
    return n


def message_log_shape(message_log: LLMMessageLogType) -> list[dict[str, Any]]:
    """Per message: the shape of every tensor value (nested message logs under list values are described recursively)."""
    out = []
    for m in message_log:
        d: dict[str, Any] = {}
        for k, v in m.items():
            if isinstance(v, torch.Tensor):
                d[k] = v.shape
            elif isinstance(v, list) and v and all(isinstance(x, list) for x in v):
                d[k] = [message_log_shape(x) for x in v]
        out.append(d)
    return out


def validate_tensor_consistency(tensors: Sequence[torch.Tensor]) -> None:
    """All tensors that will be concatenated into one row must agree in dtype and device."""
    if not tensors:
        return
    dt, dev = tensors[0].dtype, tensors[0].device
    for t in tensors[1:]:
        if t.dtype != dt or t.device != dev:
            raise ValueError(f"tensors of one message log disagree: {t.dtype} on {t.device} vs {dt} on {dev}")


def pad_tensor(t: torch.Tensor, length: int, pad_side: str = "right", pad_value=0) -> torch.Tensor:
    """Pads (never truncates) the first dimension to ``length`` on the given side."""
    n = t.shape[0]
    if n >= length:
        return t
    fill = torch.full((length - n,) + tuple(t.shape[1:]), pad_value, dtype=t.dtype, device=t.device)
    return torch.cat([t, fill]) if pad_side == "right" else torch.cat([fill, t])


def remap_dataset_keys(dataset, mapping: dict[str, str]):
    """Renames record fields (``mapping``: old -> new). Works on HuggingFace datasets (``.map``) and on lists of dicts."""
    if all(k == v for k, v in mapping.items()):
        return dataset
    if hasattr(dataset, "map") and hasattr(dataset, "column_names"):
        return dataset.map(lambda x: {v: x[k] for k, v in mapping.items()}, remove_columns=list(mapping))
    return [{**{k: v for k, v in r.items() if k not in mapping}, **{new: r[old] for old, new in mapping.items()}} for r in dataset]


# ---- a batch of message logs as a few arrays (cheap to ship through the data plane) and back
MESSAGE_LOG_BULK_FIELDS = ("turn_lengths", "turn_roles", "turn_contents")


def decompose_message_log(message_logs: Sequence[LLMMessageLogType]) -> dict[str, Any]:
    """``turn_lengths`` [B, max_turns] (0 in unused slots and for turns without tokens), ``turn_roles`` / ``turn_contents``
    (object arrays of lists) and ``response_token_lengths`` [B] (tokens of the first assistant turn, what reward shaping
    reads). Together with the flat ``input_ids`` they carry everything :func:`reconstruct_message_log` needs."""
    import numpy as np

    B = len(message_logs)
    T = max((len(ml) for ml in message_logs), default=0)
    lengths = torch.zeros((B, T), dtype=torch.long)
    roles, contents = np.empty(B, dtype=object), np.empty(B, dtype=object)
    resp = torch.zeros(B, dtype=torch.long)
    for i, ml in enumerate(message_logs):
        roles[i], contents[i] = [m["role"] for m in ml], [m.get("content", "") for m in ml]
        for t, m in enumerate(ml):
            tok = m.get("token_ids")
            if tok is None:
                continue
            n = int(tok.shape[0]) if isinstance(tok, torch.Tensor) else len(tok)
            lengths[i, t] = n
            if m["role"] == "assistant" and resp[i] == 0:
                resp[i] = n
    return {"turn_lengths": lengths, "turn_roles": roles, "turn_contents": contents, "response_token_lengths": resp}


def reconstruct_message_log(input_ids: torch.Tensor, turn_lengths: torch.Tensor, turn_roles, turn_contents,
                            generation_logprobs: Optional[torch.Tensor] = None) -> list[LLMMessageLogType]:
    """Inverse of :func:`decompose_message_log`: per-turn ``token_ids`` (and assistant ``generation_logprobs``) are VIEWS
    into the rows of ``input_ids`` / ``generation_logprobs``."""
    out = []
    for i, lens in enumerate(turn_lengths.tolist()):
        log, off = [], 0
        for t, role in enumerate(turn_roles[i]):
            n = lens[t]
            m: dict[str, Any] = {"role": role, "content": turn_contents[i][t]}
            if n:
                m["token_ids"] = input_ids[i, off : off + n]
                if generation_logprobs is not None and role == "assistant":
                    m["generation_logprobs"] = generation_logprobs[i, off : off + n]
                off += n
            log.append(m)
        out.append(log)
    return out


def attach_message_log_view(batch: BatchedDataDict) -> None:
    """Rebuilds ``batch['message_log']`` in place when the decomposed fields travelled instead of the logs themselves."""
    if "input_ids" not in batch or any(k not in batch for k in MESSAGE_LOG_BULK_FIELDS):
        return
    batch["message_log"] = reconstruct_message_log(batch["input_ids"], batch["turn_lengths"], batch["turn_roles"], batch["turn_contents"],
                                                   batch.get("generation_logprobs"))


def _with_task_prompt(content, prompt: str):
    """The task's prompt template applied to the text of a message (a string, or the text parts of a multimodal list)."""
    if isinstance(content, str):
        return prompt.format(content)
    return [dict(it, text=prompt.format(it["text"])) if it.get("type") == "text" else it for it in content]


def get_formatted_message_log(message_log: list[dict[str, Any]], tokenizer, task_data_spec=None,
                              add_bos_token: bool = True, add_eos_token: bool = True,
                              add_generation_prompt: bool = False, tools: Optional[list[dict]] = None,
                              debug: bool = False) -> LLMMessageLogType:
    """Tokenises a chat with the tokenizer's template message by message, so that every message owns exactly the text (and
    tokens) the template emits for it: the conversation is rendered up to each message and the part that is new since the
    previous rendering is that message's chunk (templates that close the previous turn differently once another one follows
    are handled by cutting at the first character that differs).

    * ``task_data_spec.system_prompt`` is put in front as a system message when the log has none; ``task_data_spec.prompt``
      (a ``str.format`` template) wraps the text of the FIRST USER message.
    * ``add_generation_prompt`` renders the assistant header as part of user / tool messages only.
    * BOS is put in front of the first chunk and EOS behind the last one unless the template already did (``<eos>`` followed
      by newlines counts as present).
    * ``tools``: tool / function definitions handed to the template.
    * multimodal content (a list of typed parts): the text parts are replaced by the chunk, the others are kept."""
    import warnings

    msgs = [dict(m) for m in message_log]
    spec = task_data_spec
    if spec is not None and getattr(spec, "system_prompt", None) and not any(m["role"] == "system" for m in msgs):
        msgs.insert(0, {"role": "system", "content": spec.system_prompt})
    if spec is not None and getattr(spec, "prompt", None):
        for m in msgs:
            if m["role"] == "user":
                m["content"] = _with_task_prompt(m["content"], spec.prompt)
                break
    out: LLMMessageLogType = []
    prev = ""
    for i, msg in enumerate(msgs):
        kw: dict[str, Any] = dict(tokenize=False, add_generation_prompt=bool(add_generation_prompt and msg["role"] in ("user", "tool")))
        if tools is not None:
            kw["tools"] = tools
        text = tokenizer.apply_chat_template(msgs[: i + 1], **kw)
        piece = text[get_first_index_that_differs(prev, text):]
        prev = text
        if debug:
            print(f"[turn {i + 1}/{len(msgs)}] role={msg['role']} chunk={piece!r}")
        if i == 0 and add_bos_token:
            if tokenizer.bos_token is None:
                warnings.warn("add_bos_token is set but the tokenizer has no BOS token")
            elif not piece.startswith(tokenizer.bos_token):
                piece = tokenizer.bos_token + piece
        if i == 0 and not add_bos_token and tokenizer.bos_token and piece.startswith(tokenizer.bos_token):
            piece = piece[len(tokenizer.bos_token):]
        if i == len(msgs) - 1 and add_eos_token:
            if tokenizer.eos_token is None:
                warnings.warn("add_eos_token is set but the tokenizer has no EOS token")
            elif not kw["add_generation_prompt"] and not piece.rstrip("\n").endswith(tokenizer.eos_token):
                piece = piece + tokenizer.eos_token
        ids = tokenizer(piece, add_special_tokens=False, return_tensors="pt")["input_ids"][0]
        new = dict(msg)
        new["token_ids"] = ids.to(torch.int64) if ids.numel() == 0 else ids     # (an empty encoding may come back as float)
        content = msg.get("content")
        if isinstance(content, list):
            new["content"] = [{"type": "text", "text": piece} if it.get("type") == "text" else it for it in content]
        else:
            new["content"] = piece
        out.append(new)
    return out
