"""Checks a rollout-routing-replay record against what the trainer's routers did (role of tools/check_r3_trace.py).

    python -m rl_b200.tools.check_r3_trace --record rollout.pt --capture train.pt [--min-agreement 0.98]

``--record``: a ``routed_experts`` tensor as the generation output carries it ([B, S, layers, k] or packed [T, layers, k] int16,
-1 where the engine has no record), or a ``{layer: [T, k]}`` dictionary written by ``rl_b200.utils.routing_trace.maybe_dump``.
``--capture``: the same for the trainer's pass over the same tokens (``RLB_R3_TRACE=<dir>`` makes the worker write them).
Reports, per MoE layer, the fraction of positions whose expert SETS agree, the fraction without a record and the most loaded
experts; exits 1 when the overall agreement is below the bound (with replay switched on it must be 1.0).
"""

from __future__ import annotations

import argparse
import json
import sys

import torch


def _as_layers(obj) -> dict[int, torch.Tensor]:
    if isinstance(obj, dict):
        return {int(k): torch.as_tensor(v).long() for k, v in obj.items()}
    t = torch.as_tensor(obj).long()
    if t.dim() == 4:
        t = t.reshape(-1, t.shape[2], t.shape[3])
    if t.dim() != 3:
        raise ValueError(f"expected [B, S, layers, k] or [T, layers, k], got {tuple(t.shape)}")
    return {j: t[:, j] for j in range(t.shape[1])}


def compare(record, capture) -> dict:
    a, b = _as_layers(record), _as_layers(capture)
    if sorted(a) != sorted(b):
        raise ValueError(f"layer sets differ: {sorted(a)} vs {sorted(b)}")
    layers, same_all, n_all = {}, 0, 0
    for j in sorted(a):
        x, y = a[j], b[j]
        if x.shape != y.shape:
            raise ValueError(f"layer {j}: shapes differ {tuple(x.shape)} vs {tuple(y.shape)}")
        have = (x >= 0).all(-1) & (y >= 0).all(-1)
        same = (x.sort(-1).values == y.sort(-1).values).all(-1) & have
        n, s = int(have.sum()), int(same.sum())
        load = torch.bincount(x[have].reshape(-1), minlength=1)
        top = load.topk(min(3, load.numel()))
        layers[j] = dict(positions=int(x.shape[0]), recorded=n, agreement=(s / n if n else 1.0), unrecorded_fraction=1 - n / max(1, x.shape[0]),
                         busiest_experts=[(int(i), int(c)) for c, i in zip(top.values, top.indices)])
        same_all, n_all = same_all + s, n_all + n
    return dict(agreement=(same_all / n_all if n_all else 1.0), recorded_positions=n_all, layers=layers)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--record", required=True)
    ap.add_argument("--capture", required=True)
    ap.add_argument("--min-agreement", type=float, default=0.98)
    a = ap.parse_args(argv)
    res = compare(torch.load(a.record, weights_only=False), torch.load(a.capture, weights_only=False))
    res["ok"] = res["agreement"] >= a.min_agreement
    print(json.dumps(res, indent=2))
    return 0 if res["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
