"""Assignment of stored samples to data-parallel ranks before a training step.

The controller balances token counts (longest-processing-time greedy) while keeping the samples of one prompt group on
one rank, so that group baselines need no communication; each rank then fetches only its own keys
(nemo_rl/data_plane/preshard.py:43).
"""

from __future__ import annotations

from typing import Sequence

from .interfaces import SampleMeta


def preshard(metas: Sequence[SampleMeta], dp_size: int, keep_groups: bool = True, equal_counts: bool = False) -> list[list[str]]:
    """Returns ``dp_size`` key lists. ``equal_counts``: every rank gets the same number of samples (required when the
    micro-batch count must match across ranks); the remainder that does not divide is left out, oldest first kept."""
    units: dict[str, list[SampleMeta]] = {}
    for m in metas:
        units.setdefault(m.group if (keep_groups and m.group is not None) else m.key, []).append(m)
    order = sorted(units.values(), key=lambda u: -sum(x.num_tokens for x in u))
    loads, counts = [0] * dp_size, [0] * dp_size
    out: list[list[str]] = [[] for _ in range(dp_size)]
    cap = None
    if equal_counts:
        total = sum(len(u) for u in order)
        cap = total // dp_size
    for u in order:
        cand = [r for r in range(dp_size) if cap is None or counts[r] + len(u) <= cap]
        if not cand:
            continue
        r = min(cand, key=lambda i: (loads[i], counts[i]))
        out[r] += [x.key for x in u]
        loads[r] += sum(x.num_tokens for x in u)
        counts[r] += len(u)
    return out
