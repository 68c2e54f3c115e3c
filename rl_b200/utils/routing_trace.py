"""Routed-expert traces: record which experts every MoE layer chose in a forward pass and replay them in another pass
(the engine's routing replayed by the trainer removes the routing mismatch between rollout and training), the role of
nemo_rl/utils/r3_trace.py and routed_experts_codec.py. ``RLB_R3_TRACE=<dir>`` makes :func:`maybe_dump` write traces."""

from __future__ import annotations

import os
from typing import Optional

import torch


def _moe_layers(model):
    return [(i, l.mlp) for i, l in enumerate(model.layers) if getattr(l, "mlp", None) is not None and hasattr(l.mlp, "last_routing")]


def capture(model) -> dict[int, torch.Tensor]:
    """Expert ids [T, k] chosen by every MoE layer in the last forward pass (int16: codec of the reference)."""
    return {i: m.last_routing.to(torch.int16).cpu() for i, m in _moe_layers(model) if m.last_routing is not None}


def replay(model, trace: Optional[dict[int, torch.Tensor]]) -> None:
    """Forces the next forward passes to use ``trace`` (``None`` clears the override)."""
    for i, m in _moe_layers(model):
        t = None if trace is None else trace.get(i)
        m.forced_routing = None if t is None else t.to(torch.int64).to(m.router.device)


def replay_rows(model, rows: Optional[torch.Tensor]) -> None:
    """``rows`` [T, MoE layers, k] (the engine's record for the T rows of the next pass, -1 where it has none): MoE layer j of
    the model is forced to ``rows[:, j]``; rows of -1 leave the choice to the router."""
    layers = _moe_layers(model)
    if rows is not None and rows.shape[1] != len(layers):
        raise ValueError(f"the routing record has {rows.shape[1]} layers, the model {len(layers)} mixture layers")
    for j, (_, m) in enumerate(layers):
        m.forced_routing = None if rows is None else rows[:, j].to(torch.int64)


def agreement(a: dict[int, torch.Tensor], b: dict[int, torch.Tensor]) -> float:
    """Fraction of (token, layer) pairs whose expert sets agree."""
    same = total = 0
    for i in a:
        if i in b and a[i].shape == b[i].shape:
            same += int((a[i].sort(-1).values == b[i].sort(-1).values).all(-1).sum())
            total += a[i].shape[0]
    return same / max(1, total)


def maybe_dump(model, step: int, tag: str = "train") -> Optional[str]:
    d = os.environ.get("RLB_R3_TRACE")
    if not d:
        return None
    os.makedirs(d, exist_ok=True)
    path = os.path.join(d, f"{tag}_step{step}.pt")
    torch.save(capture(model), path)
    return path
