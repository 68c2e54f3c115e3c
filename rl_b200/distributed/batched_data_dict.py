"""``BatchedDataDict``: a dict of batch-major tensors (and per-sample lists) with the sharding, packing and
micro-batching operations the training and generation paths need.

It plays the role of nemo_rl/distributed/batched_data_dict.py:125-1016 in the reference: shard a global batch
over data-parallel ranks, optionally re-ordering samples by length for dynamic batching or assigning them to
token-budgeted bins for sequence packing, and iterate micro-batches. The implementation keeps one rule: every
value's leading dimension is the batch dimension; python lists are treated as per-sample columns.
"""

from __future__ import annotations

from collections import UserDict
from typing import Any, Iterable, Iterator, Optional, Sequence

import torch

from rl_b200.data.packing import get_packer


def _is_batched(v: Any) -> bool:
    return isinstance(v, (torch.Tensor, list))


class BatchedDataDict(UserDict):
    """Dict whose tensor / list values share a leading batch dimension."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.micro_batch_indices: Optional[list[list[tuple[int, int]]]] = None
        self.micro_batch_lengths: Optional[list[list[int]]] = None
        self.elem_counts_per_gb: Optional[list[int]] = None

    # ------------------------------------------------------------------ basics
    @property
    def size(self) -> int:
        for v in self.data.values():
            if isinstance(v, torch.Tensor):
                return v.shape[0]
            if isinstance(v, list):
                return len(v)
        return 0

    def __len__(self) -> int:  # number of keys, like a dict
        return len(self.data)

    def to(self, device, non_blocking: bool = False) -> "BatchedDataDict":
        for k, v in self.data.items():
            if isinstance(v, torch.Tensor):
                self.data[k] = v.to(device, non_blocking=non_blocking)
        return self

    def cpu(self) -> "BatchedDataDict":
        return self.to("cpu")

    def _new_like(self) -> "BatchedDataDict":
        return type(self)()

    def select_indices(self, idx: Sequence[int] | torch.Tensor) -> "BatchedDataDict":
        out = self._new_like()
        it = idx.tolist() if isinstance(idx, torch.Tensor) else list(idx)
        tidx = torch.as_tensor(it, dtype=torch.long)
        for k, v in self.data.items():
            if isinstance(v, torch.Tensor):
                out[k] = v[tidx.to(v.device)]
            elif isinstance(v, list):
                out[k] = [v[i] for i in it]
            else:
                out[k] = v
        return out

    def slice(self, start: int, end: int) -> "BatchedDataDict":
        out = self._new_like()
        for k, v in self.data.items():
            out[k] = v[start:end] if _is_batched(v) else v
        return out

    def repeat_interleave(self, n: int) -> "BatchedDataDict":
        out = self._new_like()
        for k, v in self.data.items():
            if isinstance(v, torch.Tensor):
                out[k] = v.repeat_interleave(n, dim=0)
            elif isinstance(v, list):
                out[k] = [x for x in v for _ in range(n)]
            else:
                out[k] = v
        return out

    def truncate_tensors(self, dim: int, truncated_len: int) -> "BatchedDataDict":
        for k, v in self.data.items():
            if isinstance(v, torch.Tensor) and v.dim() > dim and v.shape[dim] > truncated_len:
                self.data[k] = v.narrow(dim, 0, truncated_len)
        return self

    def get_dict(self) -> dict:
        return dict(self.data)

    @classmethod
    def from_batches(cls, batches: Iterable[dict], pad_value_dict: Optional[dict[str, float]] = None) -> "BatchedDataDict":
        """Concatenates batches along dim 0. 2-D+ tensors whose trailing sizes differ are right-padded (per key
        pad value, default 0)."""
        batches = [b for b in batches if b is not None]
        out = cls()
        if not batches:
            return out
        pad_value_dict = pad_value_dict or {}
        for k in batches[0].keys():
            vals = [b[k] for b in batches]
            v0 = vals[0]
            if isinstance(v0, torch.Tensor):
                if v0.dim() >= 2 and len({tuple(v.shape[1:]) for v in vals}) > 1:
                    tgt = [max(v.shape[d] for v in vals) for d in range(1, v0.dim())]
                    padded = []
                    for v in vals:
                        if list(v.shape[1:]) != tgt:
                            pad = []
                            for d in range(v.dim() - 1, 0, -1):
                                pad += [0, tgt[d - 1] - v.shape[d]]
                            v = torch.nn.functional.pad(v, pad, value=pad_value_dict.get(k, 0))
                        padded.append(v)
                    vals = padded
                out[k] = torch.cat(vals, dim=0)
            elif isinstance(v0, list):
                out[k] = [x for v in vals for x in v]
            else:
                out[k] = v0
        return out

    def all_gather(self, group=None) -> "BatchedDataDict":
        """Gathers every rank's batch (python-object gather; control-plane sizes only)."""
        import torch.distributed as dist

        if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
            return self
        objs: list = [None] * dist.get_world_size(group)
        cpu = {k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in self.data.items()}
        dist.all_gather_object(objs, cpu, group=group)
        return type(self).from_batches(objs)

    # ------------------------------------------------------------------ sharding
    def shard_by_batch_size(
        self,
        shards: int,
        batch_size: Optional[int] = None,
        allow_uneven_shards: bool = False,
        dynamic_batching_args: Optional[dict] = None,
        sequence_packing_args: Optional[dict] = None,
    ):
        """Splits the batch into ``shards`` data-parallel shards.

        With ``batch_size`` (the global batch size) the data is first cut into global batches of that many
        samples and every shard receives ``batch_size / shards`` samples of each, so that all ranks step their
        optimizers the same number of times.

        ``dynamic_batching_args`` = {input_key, input_lengths_key, sequence_length_round, max_tokens_per_microbatch}:
        samples of each global batch are sorted by length before being dealt to shards, and each shard's
        micro-batches are cut so that (padded length x count) stays under the token budget.

        ``sequence_packing_args`` = {input_key, input_lengths_key, max_tokens_per_microbatch, algorithm,
        sequence_length_pad_multiple}: samples are bin-packed by length into micro-batches of at most the token
        budget; bins are dealt to shards so that every shard gets the same number of bins (ranks short of a
        bin get an empty one).

        Returns a list of ``BatchedDataDict`` (one per shard). When batching args are given each shard carries
        ``micro_batch_indices`` / ``micro_batch_lengths`` per global batch, used by ``make_microbatch_iterator_*``.
        With dynamic batching / packing the second return value maps sorted positions back to input order:
        ``(shards, sorted_indices)``.
        """
        assert not (dynamic_batching_args and sequence_packing_args), "choose dynamic batching or packing, not both"
        total = self.size
        if batch_size is None:
            batch_size = total
        if allow_uneven_shards:
            assert batch_size == total and not dynamic_batching_args and not sequence_packing_args
            base, rem = divmod(total, shards)
            out, s = [], 0
            for r in range(shards):
                n = base + (1 if r < rem else 0)
                out.append(self.slice(s, s + n))
                s += n
            return out
        assert total % batch_size == 0, f"batch of {total} samples is not a multiple of batch_size {batch_size}"
        assert batch_size % shards == 0, f"batch_size {batch_size} not divisible by {shards} shards"
        num_gb = total // batch_size
        per_shard = batch_size // shards

        if not dynamic_batching_args and not sequence_packing_args:
            idx_per_shard: list[list[int]] = [[] for _ in range(shards)]
            for g in range(num_gb):
                for r in range(shards):
                    s = g * batch_size + r * per_shard
                    idx_per_shard[r].extend(range(s, s + per_shard))
            return [self.select_indices(ix) for ix in idx_per_shard]

        args = dynamic_batching_args or sequence_packing_args
        lengths = self.data[args["input_lengths_key"]].tolist()
        budget = int(args["max_tokens_per_microbatch"])
        shard_indices: list[list[int]] = [[] for _ in range(shards)]
        shard_mb_idx: list[list[list[tuple[int, int]]]] = [[] for _ in range(shards)]
        shard_mb_len: list[list[list[int]]] = [[] for _ in range(shards)]

        if dynamic_batching_args:
            rnd = int(args.get("sequence_length_round", 1))
            for g in range(num_gb):
                gidx = list(range(g * batch_size, (g + 1) * batch_size))
                gidx.sort(key=lambda i: lengths[i])
                # deal sorted samples round-robin so every shard sees the same length profile
                per = [gidx[r::shards] for r in range(shards)]
                n_mbs = []
                cuts_all = []
                for r in range(shards):
                    cuts, lens, start = [], [], 0
                    while start < len(per[r]):
                        end = start
                        cur_max = 0
                        while end < len(per[r]):
                            L = -(-lengths[per[r][end]] // rnd) * rnd
                            new_max = max(cur_max, L)
                            if end > start and new_max * (end - start + 1) > budget:
                                break
                            cur_max = new_max
                            end += 1
                        cuts.append((start, end))
                        lens.append(cur_max)
                        start = end
                    cuts_all.append((cuts, lens))
                    n_mbs.append(len(cuts))
                for r in range(shards):
                    base = len(shard_indices[r])
                    cuts, lens = cuts_all[r]
                    shard_indices[r].extend(per[r])
                    shard_mb_idx[r].append([(base + a, base + b) for a, b in cuts])
                    shard_mb_len[r].append(lens)
        else:
            pad_mult = int(args.get("sequence_length_pad_multiple", 1))
            packer = get_packer(args.get("algorithm", "modified_first_fit_decreasing"), bin_capacity=budget,
                                collect_metrics=False, min_bin_count=shards, bin_count_multiple=shards)
            for g in range(num_gb):
                gidx = list(range(g * batch_size, (g + 1) * batch_size))
                padded = [-(-lengths[i] // pad_mult) * pad_mult for i in gidx]
                bins = packer.pack(padded)
                # bins dealt to shards; bin count is a multiple of `shards`
                per_bins = [bins[r::shards] for r in range(shards)]
                for r in range(shards):
                    base = len(shard_indices[r])
                    mb_idx, mb_len, pos = [], [], base
                    for b in per_bins[r]:
                        ids = [gidx[j] for j in b]
                        shard_indices[r].extend(ids)
                        mb_idx.append((pos, pos + len(ids)))
                        mb_len.append(sum(padded[j] for j in b))
                        pos += len(ids)
                    shard_mb_idx[r].append(mb_idx)
                    shard_mb_len[r].append(mb_len)

        out = []
        for r in range(shards):
            sh = self.select_indices(shard_indices[r])
            sh.micro_batch_indices = shard_mb_idx[r]
            sh.micro_batch_lengths = shard_mb_len[r]
            sh.elem_counts_per_gb = [sum(b - a for a, b in mbs) for mbs in shard_mb_idx[r]]
            out.append(sh)
        sorted_indices = [i for r in range(shards) for i in shard_indices[r]]
        return out, sorted_indices

    def reorder_data(self, sorted_indices: Sequence[int]) -> "BatchedDataDict":
        """Inverse of the permutation returned by ``shard_by_batch_size`` (applied to concatenated shard results)."""
        inv = [0] * len(sorted_indices)
        for pos, orig in enumerate(sorted_indices):
            inv[orig] = pos
        return self.select_indices(inv)

    # ------------------------------------------------------------------ micro-batches
    def make_microbatch_iterator(self, microbatch_size: int) -> Iterator["BatchedDataDict"]:
        n = self.size
        assert microbatch_size > 0
        for s in range(0, n, microbatch_size):
            yield self.slice(s, min(n, s + microbatch_size))

    def make_microbatch_iterator_with_dynamic_shapes(self, sequence_dim: int = 1) -> Iterator["BatchedDataDict"]:
        """Micro-batches cut by ``shard_by_batch_size(dynamic_batching_args=...)``; sequence dims trimmed to each
        micro-batch's padded length."""
        assert self.micro_batch_indices is not None
        for mbs, lens in zip(self.micro_batch_indices, self.micro_batch_lengths):
            for (a, b), L in zip(mbs, lens):
                mb = self.slice(a, b)
                mb.truncate_tensors(sequence_dim, L)
                yield mb

    def make_microbatch_iterator_for_packable_sequences(self) -> Iterator["BatchedDataDict"]:
        """Micro-batches (bins) chosen by ``shard_by_batch_size(sequence_packing_args=...)``."""
        assert self.micro_batch_indices is not None
        for mbs in self.micro_batch_indices:
            for a, b in mbs:
                yield self.slice(a, b)

    def get_microbatch_iterator_len(self) -> int:
        assert self.micro_batch_indices is not None
        return sum(len(m) for m in self.micro_batch_indices)

    def get_batch(self, batch_idx: int, batch_size: Optional[int] = None) -> "BatchedDataDict":
        """The ``batch_idx``-th global-batch slice held by this shard."""
        if self.elem_counts_per_gb is not None:
            start = sum(self.elem_counts_per_gb[:batch_idx])
            sl = self.slice(start, start + self.elem_counts_per_gb[batch_idx])
            off = start
            sl.micro_batch_indices = [[(a - off, b - off) for a, b in self.micro_batch_indices[batch_idx]]]
            sl.micro_batch_lengths = [self.micro_batch_lengths[batch_idx]]
            return sl
        assert batch_size is not None
        return self.slice(batch_idx * batch_size, (batch_idx + 1) * batch_size)
