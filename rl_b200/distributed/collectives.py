"""Small collective helpers used by the algorithms (nemo_rl/distributed/collectives.py:21-99) and the packed weight
broadcast that serves as the collective twin of refit for engines that do not share memory with the trainer
(nemo_rl/utils/packed_tensor.py:23-256)."""

from __future__ import annotations

from typing import Any, Iterable, Iterator, Optional, Sequence

import torch
import torch.distributed as dist


def rebalance_nd_tensor(t: torch.Tensor, group=None) -> torch.Tensor:
    """Ranks hold tensors that differ in their first dimension; every rank gets the concatenation over ranks (padded
    all-gather: NCCL wants equal sizes)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return t
    world = dist.get_world_size(group)
    n = torch.tensor([t.shape[0]], dtype=torch.int64, device=t.device)
    sizes = [torch.zeros_like(n) for _ in range(world)]
    dist.all_gather(sizes, n, group=group)
    sizes = [int(s) for s in sizes]
    m = max(sizes)
    pad = torch.zeros((m, *t.shape[1:]), dtype=t.dtype, device=t.device)
    pad[: t.shape[0]] = t
    parts = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(parts, pad, group=group)
    return torch.cat([p[:s] for p, s in zip(parts, sizes)], 0)


def gather_jagged_object_lists(local: list, group=None) -> list:
    """Every rank contributes a list of picklable objects; all ranks get the concatenation in rank order."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return list(local)
    box = [None] * dist.get_world_size(group)
    dist.all_gather_object(box, list(local), group=group)
    return [x for part in box for x in part]


# --------------------------------------------------------------------------------------------- packed broadcast
def pack_tensors(named: Iterable[tuple[str, torch.Tensor]], bucket_bytes: int) -> Iterator[tuple[list[tuple[str, tuple, torch.dtype, int, int]], torch.Tensor]]:
    """Groups tensors into uint8 buckets of at most ``bucket_bytes`` (a larger tensor gets a bucket of its own). Yields
    (manifest, bucket): manifest rows are (name, shape, dtype, byte offset, byte size), offsets 16-byte aligned."""
    manifest, chunks, size = [], [], 0

    def flush():
        nonlocal manifest, chunks, size
        if not manifest:
            return None
        buf = torch.empty(size, dtype=torch.uint8, device=chunks[0][1].device)
        for off, t in chunks:
            buf[off : off + t.numel() * t.element_size()] = t.contiguous().view(-1).view(torch.uint8)
        out = (manifest, buf)
        manifest, chunks, size = [], [], 0
        return out

    for name, t in named:
        nb = t.numel() * t.element_size()
        if size and size + nb > bucket_bytes:
            yield flush()
        off = -(-size // 16) * 16
        manifest.append((name, tuple(t.shape), t.dtype, off, nb))
        chunks.append((off, t))
        size = off + nb
    last = flush()
    if last is not None:
        yield last


def unpack_bucket(manifest, buf: torch.Tensor) -> Iterator[tuple[str, torch.Tensor]]:
    for name, shape, dtype, off, nb in manifest:
        yield name, buf[off : off + nb].view(dtype).view(shape)


def packed_broadcast(named: Optional[Iterable[tuple[str, torch.Tensor]]], src: int, group=None, bucket_bytes: int = 256 << 20,
                     device=None) -> Iterator[tuple[str, torch.Tensor]]:
    """The source rank streams its tensors as packed uint8 buckets; every rank (the source included) yields (name, tensor)
    views of the received bucket. Manifests travel as objects, payloads as one broadcast per bucket."""
    rank = dist.get_rank(group)
    it = pack_tensors(named, bucket_bytes) if rank == dist.get_rank(group) and named is not None else iter(())
    src_global = dist.get_global_rank(group, src) if group is not None else src
    while True:
        item = next(it, None) if rank == src else None
        head = [None if item is None else (item[0], int(item[1].numel()))]
        dist.broadcast_object_list(head, src=src_global, group=group)
        if head[0] is None:
            return
        manifest, nbytes = head[0]
        buf = item[1] if rank == src else torch.empty(nbytes, dtype=torch.uint8, device=device or "cpu")
        dist.broadcast(buf, src=src_global, group=group)
        yield from unpack_bucket(manifest, buf)
