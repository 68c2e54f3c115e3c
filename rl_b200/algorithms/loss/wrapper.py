"""Wrappers around loss functions.

* :class:`PerSequenceLossWrapper` evaluates a loss one sequence at a time (each row cut to its own length) and adds the
  results up. With globally normalised losses (every loss here divides by ``global_valid_toks`` / ``global_valid_seqs``) this
  equals one call on the whole padded batch; it is the unfused twin of the packed evaluation the policy worker does, and
  bounds the working set to one sequence when a loss materialises something of size S x V
  (nemo_rl/algorithms/loss/wrapper.py:28-166).
* :class:`DraftLossWrapper` trains a speculative-decoding draft head next to the policy: policy loss + weight x draft
  cross-entropy against the policy's detached distribution (``:231-289``).
"""

from __future__ import annotations

import math
from typing import Any, Optional

import torch

from rl_b200.distributed.batched_data_dict import BatchedDataDict

_MIN_KEYS = {"probs_ratio_min", "probs_ratio_clamped_min"}
_MAX_KEYS = {"probs_ratio_max", "probs_ratio_clamped_max"}


def merge_metrics(acc: dict, new: dict) -> dict:
    """Sums metrics across calls, except the ratio extrema, which keep their minimum / maximum (infinite values are ignored)."""
    for k, v in new.items():
        val = v.item() if isinstance(v, torch.Tensor) and v.ndim == 0 else v
        if not isinstance(val, (int, float)):
            acc[k] = val
            continue
        if k in _MIN_KEYS:
            if not math.isinf(val):
                acc[k] = min(acc.get(k, float("inf")), val)
        elif k in _MAX_KEYS:
            if not math.isinf(val):
                acc[k] = max(acc.get(k, float("-inf")), val)
        else:
            acc[k] = acc.get(k, 0) + val
    return acc


class PerSequenceLossWrapper:
    def __init__(self, loss_fn):
        self.loss_fn = loss_fn
        self.loss_type = getattr(loss_fn, "loss_type", None)
        self.input_type = getattr(loss_fn, "input_type", None)
        self.cfg = getattr(loss_fn, "cfg", None)

    def __call__(self, data: BatchedDataDict = None, global_valid_seqs=None, global_valid_toks=None, **loss_input: torch.Tensor):
        lengths = data["input_lengths"].tolist()
        total: Any = 0.0
        metrics: dict = {}
        for i, n in enumerate(lengths):
            row = {}
            for k, v in data.items():
                if isinstance(v, torch.Tensor) and v.ndim > 1 and v.shape[1] > 1:
                    row[k] = v[i : i + 1, :n]
                elif isinstance(v, torch.Tensor):
                    row[k] = v[i : i + 1]
                else:
                    row[k] = v[i : i + 1]
            # per-token inputs aligned with positions 1..S-1 (next-token quantities) are one shorter than the sequence
            inp = {k: (v[i : i + 1, : (n - 1 if v.shape[1] == data["input_ids"].shape[1] - 1 else n)] if v.ndim > 1 else v[i : i + 1])
                   for k, v in loss_input.items()}
            loss, m = self.loss_fn(data=BatchedDataDict(row), global_valid_seqs=global_valid_seqs, global_valid_toks=global_valid_toks, **inp)
            total = total + loss
            merge_metrics(metrics, m)
        return total, metrics


class DraftLossWrapper:
    """``loss = policy_loss + draft_weight * draft_cross_entropy``. The worker passes the policy loss inputs plus
    ``draft_logits`` and ``target_logits`` ([B, S-1, V], the latter detached inside the draft loss)."""

    def __init__(self, policy_loss_fn, draft_loss_fn=None, draft_weight: float = 1.0):
        from rl_b200.algorithms.loss.loss_functions import DraftCrossEntropyLossFn

        self.policy_loss_fn, self.draft_loss_fn, self.draft_weight = policy_loss_fn, draft_loss_fn or DraftCrossEntropyLossFn(), draft_weight
        self.loss_type = getattr(policy_loss_fn, "loss_type", None)
        self.input_type = getattr(policy_loss_fn, "input_type", None)
        self.cfg = getattr(policy_loss_fn, "cfg", None)
        self.needs_draft_logits = True

    def __call__(self, data=None, global_valid_seqs=None, global_valid_toks=None, draft_logits: Optional[torch.Tensor] = None,
                 target_logits: Optional[torch.Tensor] = None, draft_token_mask: Optional[torch.Tensor] = None, **loss_input):
        loss, metrics = self.policy_loss_fn(data=data, global_valid_seqs=global_valid_seqs, global_valid_toks=global_valid_toks, **loss_input)
        if draft_logits is None:
            return loss, metrics
        d_loss, d_metrics = self.draft_loss_fn(draft_logits, target_logits, data, global_valid_seqs, global_valid_toks,
                                               **({"token_mask": draft_token_mask} if draft_token_mask is not None else {}))
        metrics = dict(metrics)
        metrics.update({("draft_" + k if not k.startswith("draft") else k): v for k, v in d_metrics.items() if k != "num_valid_samples"})
        metrics["policy_loss"] = metrics.get("loss")
        total = loss + self.draft_weight * d_loss
        metrics["loss"] = float(total.item())
        return total, metrics
