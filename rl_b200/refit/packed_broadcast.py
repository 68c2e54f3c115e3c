"""Packed broadcast: many tensors travel as a few large byte buffers, one collective each.

``broadcast_packed`` is the generic tool (the role of nemo_rl/utils/packed_tensor.py:39-256: pack into uint8 buckets,
broadcast, unpack on the receivers). ``PipelineWeightSynchronizer`` uses it to give every rank of a pipeline-parallel
trainer a complete serving copy of the model: each stage broadcasts the tensors it owns over the pipeline group, and all
ranks write them into their serving model (which keeps the trainer's tensor-parallel layout).
"""

from __future__ import annotations

from typing import Callable, Iterable, Iterator, Optional

import torch
import torch.distributed as dist

DEFAULT_BUCKET_BYTES = 256 << 20


def _buckets(items: Iterable[tuple[str, torch.Tensor]], bucket_bytes: int) -> Iterator[list[tuple[str, torch.Tensor]]]:
    cur, size = [], 0
    for name, t in items:
        nb = t.numel() * t.element_size()
        if cur and size + nb > bucket_bytes:
            yield cur
            cur, size = [], 0
        cur.append((name, t))
        size += nb
    if cur:
        yield cur


def pack(tensors: list[torch.Tensor], device) -> torch.Tensor:
    """Concatenates the raw bytes of ``tensors`` (each padded to 16 bytes) into one uint8 buffer on ``device``."""
    total = sum(-(-t.numel() * t.element_size() // 16) * 16 for t in tensors)
    buf = torch.empty(total, dtype=torch.uint8, device=device)
    off = 0
    for t in tensors:
        nb = t.numel() * t.element_size()
        buf[off : off + nb].copy_(t.detach().contiguous().view(-1).view(torch.uint8))
        off += -(-nb // 16) * 16
    return buf


def unpack(buf: torch.Tensor, meta: list[tuple[str, tuple, torch.dtype]]) -> Iterator[tuple[str, torch.Tensor]]:
    off = 0
    for name, shape, dtype in meta:
        n = 1
        for s in shape:
            n *= s
        nb = n * torch.empty((), dtype=dtype).element_size()
        yield name, buf[off : off + nb].view(dtype).view(shape)
        off += -(-nb // 16) * 16


def broadcast_packed(items: Optional[Iterable[tuple[str, torch.Tensor]]], src: int, group, consume: Callable[[str, torch.Tensor], None],
                     device, bucket_bytes: int = DEFAULT_BUCKET_BYTES) -> int:
    """The rank whose *group* rank is ``src`` provides ``items``; every rank of ``group`` (the source included) gets each
    (name, tensor) through ``consume``. Returns the number of payload bytes. Collective over ``group``."""
    me = dist.get_rank(group)
    g_src = dist.get_global_rank(group, src) if group is not None else src
    total = 0
    it = _buckets(items, bucket_bytes) if me == src else None
    while True:
        if me == src:
            bucket = next(it, None)
            head = [None if bucket is None else [(n, tuple(t.shape), t.dtype) for n, t in bucket]]
        else:
            bucket, head = None, [None]
        dist.broadcast_object_list(head, src=g_src, group=group)
        meta = head[0]
        if meta is None:
            return total
        if me == src:
            buf = pack([t for _, t in bucket], device)
        else:
            size = sum(-(-_numel(s) * torch.empty((), dtype=d).element_size() // 16) * 16 for _, s, d in meta)
            buf = torch.empty(size, dtype=torch.uint8, device=device)
        dist.broadcast(buf, src=g_src, group=group)
        total += buf.numel()
        for name, t in unpack(buf, meta):
            consume(name, t)


def _numel(shape) -> int:
    n = 1
    for s in shape:
        n *= s
    return n


class PipelineWeightSynchronizer:
    """Serving copy of the whole model on every rank of a pipeline-parallel trainer (same tensor-parallel layout)."""

    def __init__(self, train_model, cfg, pstate, bucket_bytes: int = DEFAULT_BUCKET_BYTES):
        from rl_b200.models.hf_io import iter_hf_shards
        from rl_b200.refit.plan import serving_param_layout
        from rl_b200.refit.synchronizer import build_serving_model

        self.train_model, self.cfg, self.st, self.bucket_bytes = train_model, cfg, pstate, bucket_bytes
        p0 = next(train_model.parameters())
        self.device, self.dtype = p0.device, p0.dtype
        tp = train_model.tp
        _, numel = serving_param_layout(cfg, tp.world)
        self.arena = torch.zeros(numel, dtype=self.dtype, device=self.device)
        self.serving_model = build_serving_model(cfg, tp.world, tp.rank, self.arena, tp.group, getattr(tp, "comm", None))
        self._dst = {hf: (dst, hs) for hf, dst, hs in iter_hf_shards(self.serving_model)}
        self.last_bytes = 0

    @torch.no_grad()
    def _consume(self, name: str, t: torch.Tensor) -> None:
        dst, hs = self._dst[name]
        if hs is not None:
            t = t.narrow(hs[0], hs[1], hs[2])
        dst.copy_(t.to(dst.dtype))

    @torch.no_grad()
    def sync_weights(self, timer=None) -> None:
        from rl_b200.models.hf_io import iter_hf_tensors

        st = self.st
        total = 0
        for stage in range(st.pp):
            # the tensor-parallel ranks of the source stage assemble full tensors together; every rank of the stage then
            # feeds its own pipeline group (the ranks with the same data / tensor coordinates on the other stages)
            items = iter_hf_tensors(self.train_model) if st.pp_rank == stage else None
            total += broadcast_packed(items, stage, st.pp_group, self._consume, self.device, self.bucket_bytes)
        self.last_bytes = total

    def close(self) -> None:
        pass
