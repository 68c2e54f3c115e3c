"""Sequence packers: assign variable-length sequences to bins of a fixed token capacity.

Algorithms offered (the set of nemo_rl/data/packing/algorithms.py:288-655): concatenative, first-fit, first-fit
decreasing, first-fit shuffle and modified first-fit decreasing (Johnson & Garey's MFFD, which places the large /
medium / small classes in a fixed order and reaches 71/60 OPT + 1 bins). Every packer returns a list of bins, each
a list of indices into the input. ``min_bin_count`` / ``bin_count_multiple`` let the caller ask for a bin count
that divides evenly over data-parallel ranks; bins are split (largest first) or empty bins appended to reach it.
"""

from __future__ import annotations

import random
from dataclasses import dataclass, field
from typing import Optional, Sequence


@dataclass
class PackingMetrics:
    """Running statistics over ``pack`` calls."""

    total_sequences: int = 0
    total_bins: int = 0
    total_tokens: int = 0
    total_capacity: int = 0
    min_utilization: float = 1.0
    max_utilization: float = 0.0
    calls: int = 0

    def update(self, lengths: Sequence[int], bins: list[list[int]], capacity: int) -> dict:
        used = [sum(lengths[i] for i in b) for b in bins]
        n = len(bins)
        self.calls += 1
        self.total_sequences += len(lengths)
        self.total_bins += n
        self.total_tokens += sum(used)
        self.total_capacity += n * capacity
        utils = [u / capacity for u in used] or [0.0]
        self.min_utilization = min(self.min_utilization, min(utils))
        self.max_utilization = max(self.max_utilization, max(utils))
        return {
            "num_bins": n,
            "avg_utilization": sum(utils) / len(utils),
            "waste_ratio": 1.0 - (sum(used) / (n * capacity) if n else 0.0),
        }

    def aggregated(self) -> dict:
        return {
            "total_sequences": self.total_sequences,
            "total_bins": self.total_bins,
            "avg_utilization": self.total_tokens / self.total_capacity if self.total_capacity else 0.0,
            "avg_sequences_per_bin": self.total_sequences / self.total_bins if self.total_bins else 0.0,
            "min_utilization": self.min_utilization,
            "max_utilization": self.max_utilization,
        }


class SequencePacker:
    name = "base"

    def __init__(self, bin_capacity: int, collect_metrics: bool = False, min_bin_count: Optional[int] = None,
                 bin_count_multiple: Optional[int] = None, seed: int = 0):
        if bin_capacity <= 0:
            raise ValueError("bin_capacity must be positive")
        self.bin_capacity = int(bin_capacity)
        self.min_bin_count = min_bin_count
        self.bin_count_multiple = bin_count_multiple
        self.metrics = PackingMetrics() if collect_metrics else None
        self.rng = random.Random(seed)

    def _check(self, lengths: Sequence[int]) -> None:
        for i, L in enumerate(lengths):
            if L > self.bin_capacity:
                raise ValueError(f"sequence {i} of length {L} exceeds the bin capacity {self.bin_capacity}")

    def _pack(self, lengths: Sequence[int]) -> list[list[int]]:
        raise NotImplementedError

    def pack(self, lengths: Sequence[int]) -> list[list[int]]:
        lengths = [int(x) for x in lengths]
        self._check(lengths)
        bins = [b for b in self._pack(lengths) if b]
        bins = self._adjust_bin_count(bins, lengths)
        if self.metrics is not None:
            self.metrics.update(lengths, bins, self.bin_capacity)
        return bins

    def _adjust_bin_count(self, bins: list[list[int]], lengths: Sequence[int]) -> list[list[int]]:
        target = len(bins)
        if self.min_bin_count:
            target = max(target, self.min_bin_count)
        if self.bin_count_multiple:
            m = self.bin_count_multiple
            target = -(-target // m) * m
        while len(bins) < target:
            # split the bin with the most sequences; when nothing can be split, pad with empty bins
            cand = max(range(len(bins)), key=lambda j: len(bins[j])) if bins else None
            if cand is None or len(bins[cand]) < 2:
                bins.append([])
                continue
            b = bins[cand]
            b.sort(key=lambda i: -lengths[i])
            bins[cand] = b[0::2]
            bins.append(b[1::2])
        return bins


class ConcatenativePacker(SequencePacker):
    """Fills bins in input order; a new bin starts when the next sequence does not fit."""

    name = "concatenative"

    def _pack(self, lengths):
        bins, cur, used = [], [], 0
        for i, L in enumerate(lengths):
            if cur and used + L > self.bin_capacity:
                bins.append(cur)
                cur, used = [], 0
            cur.append(i)
            used += L
        if cur:
            bins.append(cur)
        return bins


def _first_fit(order: Sequence[int], lengths: Sequence[int], cap: int) -> list[list[int]]:
    bins: list[list[int]] = []
    room: list[int] = []
    for i in order:
        L = lengths[i]
        for j, r in enumerate(room):
            if L <= r:
                bins[j].append(i)
                room[j] -= L
                break
        else:
            bins.append([i])
            room.append(cap - L)
    return bins


class FirstFitPacker(SequencePacker):
    name = "first_fit"

    def _pack(self, lengths):
        return _first_fit(range(len(lengths)), lengths, self.bin_capacity)


class FirstFitDecreasingPacker(SequencePacker):
    name = "first_fit_decreasing"

    def _pack(self, lengths):
        order = sorted(range(len(lengths)), key=lambda i: -lengths[i])
        return _first_fit(order, lengths, self.bin_capacity)


class FirstFitShufflePacker(SequencePacker):
    name = "first_fit_shuffle"

    def _pack(self, lengths):
        order = list(range(len(lengths)))
        self.rng.shuffle(order)
        return _first_fit(order, lengths, self.bin_capacity)


class ModifiedFirstFitDecreasingPacker(SequencePacker):
    """Johnson & Garey's MFFD.

    Items are classed by size relative to the capacity C: large (> C/2), medium (> C/3), small (> C/6), tiny.
    1. every large item opens a bin (largest first);
    2. going through those bins from the emptiest-room... in order, each receives the largest medium item that fits;
    3. going through the bins without a medium item in reverse order, a bin receives the two smallest small items
       if they fit together, then the smallest is swapped for the largest small item that still fits;
    4. going forward again, each bin greedily takes the largest remaining small / tiny item that fits;
    5. whatever is left is packed first-fit-decreasing into new bins.
    """

    name = "modified_first_fit_decreasing"

    def _pack(self, lengths):
        C = self.bin_capacity
        idx = sorted(range(len(lengths)), key=lambda i: -lengths[i])
        large = [i for i in idx if lengths[i] > C / 2]
        medium = [i for i in idx if C / 3 < lengths[i] <= C / 2]
        small = [i for i in idx if C / 6 < lengths[i] <= C / 3]
        tiny = [i for i in idx if lengths[i] <= C / 6]

        bins = [[i] for i in large]
        room = [C - lengths[i] for i in large]
        has_medium = [False] * len(bins)

        # step 2: forward, largest medium that fits
        for j in range(len(bins)):
            for k, i in enumerate(medium):
                if lengths[i] <= room[j]:
                    bins[j].append(i)
                    room[j] -= lengths[i]
                    has_medium[j] = True
                    medium.pop(k)
                    break

        # step 3: backward over bins without a medium item, pairs of small items
        for j in range(len(bins) - 1, -1, -1):
            if has_medium[j] or len(small) < 2:
                continue
            a, b = small[-1], small[-2]  # the two smallest
            if lengths[a] + lengths[b] > room[j]:
                continue
            small.pop()  # take the smallest
            bins[j].append(a)
            room[j] -= lengths[a]
            for k, i in enumerate(small):  # largest that still fits
                if lengths[i] <= room[j]:
                    bins[j].append(i)
                    room[j] -= lengths[i]
                    small.pop(k)
                    break

        # step 4: forward, greedily the largest remaining item that fits
        rest = sorted(medium + small + tiny, key=lambda i: -lengths[i])
        for j in range(len(bins)):
            k = 0
            while k < len(rest):
                i = rest[k]
                if lengths[i] <= room[j]:
                    bins[j].append(i)
                    room[j] -= lengths[i]
                    rest.pop(k)
                else:
                    k += 1

        # step 5: first-fit decreasing for the remainder
        bins.extend(_first_fit(rest, lengths, C))
        return bins


_PACKERS = {
    p.name: p
    for p in (ConcatenativePacker, FirstFitPacker, FirstFitDecreasingPacker, FirstFitShufflePacker,
              ModifiedFirstFitDecreasingPacker)
}


def get_packer(algorithm: str, bin_capacity: int, collect_metrics: bool = False, min_bin_count: Optional[int] = None,
               bin_count_multiple: Optional[int] = None, seed: int = 0) -> SequencePacker:
    key = str(algorithm).lower()
    if key not in _PACKERS:
        raise ValueError(f"unknown packing algorithm '{algorithm}'; choose from {sorted(_PACKERS)}")
    return _PACKERS[key](bin_capacity, collect_metrics, min_bin_count, bin_count_multiple, seed)
