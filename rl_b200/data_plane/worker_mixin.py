"""Worker side of the data plane: fetch the assigned keys once per model-parallel group and share them inside it.

Ranks of one tensor- / context-parallel group train on the same samples, so only the group's first rank talks to the
store; the batch then travels over the group's own links (nemo_rl/data_plane/worker_mixin.py:53-122).
"""

from __future__ import annotations

from typing import Iterable, Optional, Sequence

import torch.distributed as dist

from rl_b200.distributed.batched_data_dict import BatchedDataDict

from .codec import records_to_batch
from .interfaces import DataPlaneClient


def fetch_batch(client: Optional[DataPlaneClient], keys: Sequence[str], fields: Optional[Iterable[str]] = None, group=None,
                pad_values: Optional[dict] = None) -> BatchedDataDict:
    """``group``: the model-parallel group sharing the data (None: this rank fetches for itself). Ranks other than the
    group's first may pass ``client=None``."""
    if group is None or dist.get_world_size(group) == 1:
        return records_to_batch(client.get(keys, fields), pad_values)
    first = dist.get_global_rank(group, 0)
    box = [None]
    if dist.get_rank() == first:
        box[0] = client.get(keys, fields)
    dist.broadcast_object_list(box, src=first, group=group)
    return records_to_batch(box[0], pad_values)


def write_back(client: Optional[DataPlaneClient], keys: Sequence[str], batch: BatchedDataDict, fields: Iterable[str], lengths=None, group=None) -> None:
    """Stores per-sample results (log-probabilities, advantages) under the samples' keys; one writer per group."""
    if group is not None and dist.get_world_size(group) > 1 and dist.get_rank() != dist.get_global_rank(group, 0):
        return
    for i, k in enumerate(keys):
        rec = {}
        for f in fields:
            v = batch[f][i]
            rec[f] = v[: int(lengths[i])].clone() if (lengths is not None and hasattr(v, "dim") and v.dim() >= 1) else v
        client.update(k, rec)
