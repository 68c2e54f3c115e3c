"""Named N-dimensional rank layouts (``NamedSharding``), the role of nemo_rl/distributed/named_sharding.py.

A layout is an integer array of ranks with a name per axis, e.g. ``[pp, dp, cp, tp]``. It answers "which ranks share
my data-parallel index", "what are my coordinates", and builds the process groups of each axis.
"""

from __future__ import annotations

import itertools
from typing import Optional, Sequence

import numpy as np


class NamedSharding:
    def __init__(self, layout, names: Sequence[str]):
        self.layout = np.asarray(layout, dtype=np.int64)
        self.names = list(names)
        if self.layout.ndim != len(self.names):
            raise ValueError(f"layout has {self.layout.ndim} axes but {len(self.names)} names were given")
        flat = self.layout.reshape(-1)
        if len(set(flat.tolist())) != flat.size:
            raise ValueError("every rank must appear exactly once in the layout")
        self._coords = {int(r): tuple(int(c) for c in idx) for idx, r in np.ndenumerate(self.layout)}

    @classmethod
    def from_sizes(cls, world: int, **sizes: int) -> "NamedSharding":
        """Row-major layout with the given axis sizes (first name = slowest axis), e.g. ``from_sizes(8, dp=2, tp=4)``."""
        names = list(sizes)
        shape = [int(sizes[n]) for n in names]
        if int(np.prod(shape)) != world:
            raise ValueError(f"axis sizes {sizes} do not multiply to the world size {world}")
        return cls(np.arange(world).reshape(shape), names)

    @property
    def shape(self) -> dict[str, int]:
        return {n: int(s) for n, s in zip(self.names, self.layout.shape)}

    @property
    def size(self) -> int:
        return int(self.layout.size)

    def get_axis_size(self, name: str) -> int:
        return int(self.layout.shape[self.names.index(name)])

    def get_worker_coords(self, rank: int) -> dict[str, int]:
        return dict(zip(self.names, self._coords[int(rank)]))

    def get_ranks(self, **fixed: int):
        """Ranks at the given coordinates; unspecified axes are kept (returns an int when all axes are fixed)."""
        idx = tuple(fixed.get(n, slice(None)) for n in self.names)
        sub = self.layout[idx]
        return int(sub) if np.ndim(sub) == 0 else sub.reshape(-1).tolist()

    def get_ranks_by_coord(self, **fixed: int) -> list[int]:
        r = self.get_ranks(**fixed)
        return [r] if isinstance(r, int) else r

    def axis_groups(self, name: str) -> list[list[int]]:
        """All rank groups that vary only along ``name`` (one process group each)."""
        ax = self.names.index(name)
        moved = np.moveaxis(self.layout, ax, -1)
        return [g.tolist() for g in moved.reshape(-1, moved.shape[-1])]

    def group_of(self, rank: int, name: str) -> list[int]:
        c = self.get_worker_coords(rank)
        c.pop(name)
        return self.get_ranks_by_coord(**c)

    def build_process_groups(self, name: str, backend: Optional[str] = None):
        """Creates every process group of axis ``name`` (all ranks must call this) and returns this rank's group."""
        import torch.distributed as dist

        mine = None
        me = dist.get_rank()
        for ranks in self.axis_groups(name):
            g = dist.new_group(ranks=ranks, backend=backend)
            if me in ranks:
                mine = g
        return mine

    def __repr__(self):
        return f"NamedSharding({self.shape})"
