"""Train-side top-k / top-p filtering so that training log-probabilities match the sampler's processed distribution
(nemo_rl/algorithms/logits_sampling_utils.py:30-285).

``apply_top_k_top_p`` masks logits outside the kept set with -inf; the mask is found without a full sort when only
top-k is active, and in vocabulary chunks of rows for top-p to bound memory. Gradients flow only through kept
entries (the masked positions receive zero gradient, as a custom backward would give).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class TrainingSamplingParams:
    top_k: Optional[int] = None
    top_p: float = 1.0
    temperature: float = 1.0

    @property
    def needs_filtering(self) -> bool:
        return (self.top_k is not None and self.top_k > 0) or self.top_p < 1.0


def need_top_k_or_top_p_filtering(top_k: Optional[int], top_p: Optional[float]) -> bool:
    return (top_k is not None and top_k > 0) or (top_p is not None and top_p < 1.0)


def apply_top_k_top_p(logits: torch.Tensor, top_k: Optional[int] = None, top_p: Optional[float] = None,
                      chunk_rows: int = 4096) -> tuple[torch.Tensor, torch.Tensor]:
    """Returns (filtered logits with -inf outside the kept set, boolean keep mask). ``logits`` [..., V]."""
    V = logits.shape[-1]
    flat = logits.reshape(-1, V)
    keep = torch.ones_like(flat, dtype=torch.bool)
    if top_k is not None and 0 < top_k < V:
        kth = torch.topk(flat.detach(), top_k, dim=-1).values[:, -1:]
        keep &= flat.detach() >= kth
    if top_p is not None and top_p < 1.0:
        for s in range(0, flat.shape[0], chunk_rows):
            z = flat[s : s + chunk_rows].detach().float().masked_fill(~keep[s : s + chunk_rows], float("-inf"))
            sz, si = torch.sort(z, dim=-1, descending=True)
            p = torch.softmax(sz, dim=-1)
            drop_sorted = (p.cumsum(-1) - p) >= top_p
            drop = torch.zeros_like(drop_sorted).scatter(-1, si, drop_sorted)
            keep[s : s + chunk_rows] &= ~drop
    out = flat.masked_fill(~keep, float("-inf"))
    return out.view_as(logits), keep.view_as(logits)


def filtered_log_softmax(logits: torch.Tensor, params: TrainingSamplingParams) -> torch.Tensor:
    """log_softmax(logits / T) after top-k / top-p, -inf outside the kept set."""
    z = logits.float() / (params.temperature if params.temperature > 0 else 1.0)
    if params.needs_filtering:
        z, _ = apply_top_k_top_p(z, params.top_k, params.top_p)
    return torch.log_softmax(z, dim=-1)
