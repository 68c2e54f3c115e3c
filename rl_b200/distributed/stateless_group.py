"""A process group outside the default ``torch.distributed`` world: rendez-vous on a TCP store, then object / tensor
exchange between an arbitrary set of processes (a trainer and an inference server that are not ranks of one job, for
instance). Role of nemo_rl/distributed/stateless_process_group.py:42-155, which wraps nccl4py the same way; here the
payload moves through the store itself (control-plane sizes) and bulk tensors use ``torch.distributed`` sub-worlds or
CUDA IPC as the caller chooses."""

from __future__ import annotations

import pickle
from datetime import timedelta
from typing import Any, Optional

import torch


class StatelessProcessGroup:
    def __init__(self, master_address: str, port: int, rank: int, world_size: int, timeout_s: float = 60.0, store=None):
        import torch.distributed as dist

        self.rank, self.world_size = rank, world_size
        self.store = store or dist.TCPStore(master_address, port, world_size, rank == 0, timeout=timedelta(seconds=timeout_s),
                                            wait_for_workers=False)
        self._seq = 0
        self._bar = 0

    def _key(self, tag: str, src: int) -> str:
        return f"slpg/{tag}/{self._seq}/{src}"

    def broadcast_obj(self, obj: Any, src: int = 0) -> Any:
        key = self._key("bc", src)
        self._seq += 1
        if self.rank == src:
            self.store.set(key, pickle.dumps(obj))
            return obj
        return pickle.loads(self.store.get(key))

    def all_gather_obj(self, obj: Any) -> list:
        seq = self._seq
        self._seq += 1
        self.store.set(f"slpg/ag/{seq}/{self.rank}", pickle.dumps(obj))
        return [pickle.loads(self.store.get(f"slpg/ag/{seq}/{r}")) for r in range(self.world_size)]

    def barrier(self) -> None:
        self._bar += 1
        key = f"slpg/bar/{self._bar}"
        self.store.add(key, 1)
        import time

        t0 = time.time()
        while int(self.store.add(key, 0)) < self.world_size:
            if time.time() - t0 > 600:
                raise TimeoutError("stateless barrier timed out")
            time.sleep(0.001)

    def broadcast_tensor(self, t: Optional[torch.Tensor], src: int = 0) -> torch.Tensor:
        """Small tensors only (metadata, scales, a few MB): serialised through the store."""
        from rl_b200.data_plane.codec import decode_record, encode_record

        key = self._key("bt", src)
        self._seq += 1
        if self.rank == src:
            self.store.set(key, encode_record({"t": t}))
            return t
        return decode_record(bytes(self.store.get(key)))["t"]

    # Rank 0 hosts the store: it must keep this object alive until every member is done with the group.

    def bulk_group(self, device=None, timeout_s: float = 1800.0):
        """A ``torch.distributed`` backend object (NCCL for CUDA tensors, gloo otherwise) over this group's members, built
        straight on the group's store: bulk tensors (weights) move through it while the default process group of either side
        is left alone. Every member must call this once, with the same kind of device."""
        if getattr(self, "_bulk", None) is None:
            import torch.distributed as dist

            store = dist.PrefixStore("slpg_bulk", self.store)
            dev = torch.device(device) if device is not None else torch.device("cpu")
            if dev.type == "cuda":
                self._bulk = dist.ProcessGroupNCCL(store, self.rank, self.world_size, timedelta(seconds=timeout_s))
            else:
                self._bulk = dist.ProcessGroupGloo(store, self.rank, self.world_size, timedelta(seconds=timeout_s))
        return self._bulk

    def broadcast_bulk(self, t: torch.Tensor, src: int = 0) -> torch.Tensor:
        """In-place broadcast of a (large) tensor from ``src`` to every member over :meth:`bulk_group`."""
        import torch.distributed as dist

        opts = dist.BroadcastOptions()
        opts.rootRank, opts.rootTensor = src, 0
        self.bulk_group(t.device).broadcast([t], opts).wait()
        return t

    def unique_id(self) -> bytes:
        """A 128-byte token agreed by all members (what a communicator bootstrap needs)."""
        import os

        return self.broadcast_obj(os.urandom(128) if self.rank == 0 else None, 0)
