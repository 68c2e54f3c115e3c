"""One entry point for every way the engine gets the trainer's weights.

``create_weight_synchronizer(kind, ...)`` returns an object with ``sync_weights()`` (and ``close()``); ``kind``:

* ``colocated``   -- trainer and engine address the same buffers: nothing to move (:class:`ColocatedHandoff`)
* ``peer``        -- re-shard over peer memory with the copy / quantising kernels (:class:`rl_b200.refit.synchronizer.WeightSynchronizer`)
* ``collective``  -- packed broadcasts over a process group (:class:`rl_b200.refit.packed_broadcast.PipelineWeightSynchronizer`, the NCCL / gloo form)
* ``sparse_tcp`` / ``sparse_http`` / ``sparse_object_store`` -- lossless xor-deltas against what the receivers hold, streamed to
  engines that share no NVLink with the trainer (:mod:`rl_b200.refit.sparse_transport`)

The reference selects among its IPC, collective, HTTP, Megatron, checkpoint-engine and nccl_reshard synchronizers the same way
(nemo_rl/weight_sync/*_weight_synchronizer.py and their factory).
"""

from __future__ import annotations

import itertools
from typing import Any, Optional


class ColocatedHandoff:
    """Matching layouts on the same GPU: the engine reads the trainer's parameters in place."""

    def __init__(self, train_model):
        self.serving_model = train_model
        self.last_bytes = 0

    def sync_weights(self, timer=None) -> None:
        return None

    def close(self) -> None:
        return None


class SparseDeltaSynchronizer:
    """Sender side of the sparse-delta refit: keeps the baseline the receivers hold and streams ``new XOR baseline``."""

    def __init__(self, train_model, transport, store=None, post=None):
        from rl_b200.models.hf_io import iter_hf_tensors
        from rl_b200.refit import sparse_transport as ST

        self.model, self.transport, self.store, self.post = train_model, transport, store, post
        self._ST, self._iter = ST, iter_hf_tensors
        self.baseline = ST.init_baseline((n, t) for n, t in iter_hf_tensors(train_model))
        self._seq = itertools.count(1)
        self.last_stats: dict = {}

    def sync_weights(self, timer=None) -> dict:
        ST, tr = self._ST, self.transport
        tid = f"refit-{next(self._seq):06d}"
        tensors = ((n, t.detach()) for n, t in self._iter(self.model))
        kw = dict(bucket_bytes=tr.bucket_bytes, encode_workers=tr.encode_workers, send_workers=tr.send_workers, level=tr.compression_level)
        if tr.kind in ("tcp", "sparse_tcp"):
            self.last_stats = ST.stream_via_tcp(tensors, self.baseline, [tuple(e) for e in tr.endpoints], tid, **kw)
        elif tr.kind in ("http", "sparse_http"):
            self.last_stats = ST.stream_via_http(tensors, self.baseline, tr, tid, post=self.post)
        elif tr.kind in ("object_store", "sparse_object_store"):
            store = self.store or ST.FileObjectStore(tr.store_dir)
            self.last_stats = ST.stream_via_manifest(tensors, self.baseline, store, tid, **kw)
        else:
            raise ValueError(f"unknown sparse transport '{tr.kind}'")
        return self.last_stats

    def close(self) -> None:
        return None


def create_weight_synchronizer(kind: str, train_model, cfg=None, *, tp_serve: Optional[int] = None, group=None, pstate=None,
                               transport: Any = None, **kw):
    kind = (kind or "colocated").lower()
    if kind == "colocated":
        return ColocatedHandoff(train_model)
    if kind in ("peer", "nccl_reshard", "reshard"):
        from rl_b200.refit.synchronizer import WeightSynchronizer

        return WeightSynchronizer(train_model, cfg, int(tp_serve or train_model.tp.world), group=group, **kw)
    if kind in ("collective", "broadcast"):
        from rl_b200.refit.packed_broadcast import PipelineWeightSynchronizer

        return PipelineWeightSynchronizer(train_model, cfg, pstate, **kw)
    if kind.startswith("sparse"):
        from rl_b200.refit.sparse_transport import SparseRefitTransport

        tr = transport if transport is not None else SparseRefitTransport(kind=kind.replace("sparse_", ""), **kw)
        return SparseDeltaSynchronizer(train_model, tr, store=kw.get("store"), post=kw.get("post"))
    raise ValueError(f"unknown weight synchronizer '{kind}' (colocated | peer | collective | sparse_tcp | sparse_http | sparse_object_store)")
