"""Process-wide parallel layout: which ranks form this rank's tensor / data / expert / pipeline / context groups.

``init_parallel(tp=, pp=, cp=, ep=)`` carves the world into a ``[pp, dp, cp, tp]`` grid (tp fastest, so tensor-parallel
ranks are NVLink neighbours), builds one process group per axis and stores them in a module-level
:class:`ParallelState` that models, the optimizer and the workers read. Expert parallelism reuses the data-parallel
(x context-parallel) ranks of a pipeline stage, as Megatron does (nemo_rl/models/megatron/setup.py:888-1023).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

import torch.distributed as dist

from rl_b200.distributed.named_sharding import NamedSharding


@dataclass
class ParallelState:
    world: int = 1
    rank: int = 0
    tp: int = 1
    pp: int = 1
    cp: int = 1
    dp: int = 1
    ep: int = 1
    tp_rank: int = 0
    pp_rank: int = 0
    cp_rank: int = 0
    dp_rank: int = 0
    ep_rank: int = 0
    sequence_parallel: bool = False
    tp_group: Any = None
    pp_group: Any = None
    cp_group: Any = None
    dp_group: Any = None
    ep_group: Any = None
    dp_cp_group: Any = None       # gradient reduction / optimizer sharding for dense parameters
    model_group: Any = None       # tp x pp x cp ranks of one data-parallel replica
    sharding: Optional[NamedSharding] = None
    tp_comm: Any = None           # fused peer-memory kernels of the tp group (GPU only)
    ep_comm: Any = None
    extras: dict = field(default_factory=dict)

    @property
    def is_first_stage(self) -> bool:
        return self.pp_rank == 0

    @property
    def is_last_stage(self) -> bool:
        return self.pp_rank == self.pp - 1


_STATE = ParallelState()


def get_state() -> ParallelState:
    return _STATE


def reset_parallel() -> None:
    global _STATE
    _STATE = ParallelState()


def init_parallel(tp: int = 1, pp: int = 1, cp: int = 1, ep: int = 1, sequence_parallel: bool = False,
                  backend: Optional[str] = None) -> ParallelState:
    """Collective: every rank of the default group must call it with the same sizes."""
    global _STATE
    if not (dist.is_available() and dist.is_initialized()):
        if tp * pp * cp * ep != 1:
            raise RuntimeError("model parallelism needs an initialised process group")
        _STATE = ParallelState()
        return _STATE
    world, rank = dist.get_world_size(), dist.get_rank()
    if world % (tp * pp * cp):
        raise ValueError(f"world size {world} is not divisible by tp*pp*cp = {tp * pp * cp}")
    dp = world // (tp * pp * cp)
    if (dp * cp) % ep:
        raise ValueError(f"expert parallel size {ep} must divide dp*cp = {dp * cp}")
    ns = NamedSharding.from_sizes(world, pp=pp, dp=dp, cp=cp, tp=tp)
    c = ns.get_worker_coords(rank)
    st = ParallelState(world=world, rank=rank, tp=tp, pp=pp, cp=cp, dp=dp, ep=ep, tp_rank=c["tp"], pp_rank=c["pp"],
                       cp_rank=c["cp"], dp_rank=c["dp"], sequence_parallel=bool(sequence_parallel and tp > 1), sharding=ns)
    st.tp_group = ns.build_process_groups("tp", backend) if tp > 1 else None
    st.pp_group = ns.build_process_groups("pp", backend) if pp > 1 else None
    st.cp_group = ns.build_process_groups("cp", backend) if cp > 1 else None
    st.dp_group = ns.build_process_groups("dp", backend) if (dp > 1 and dp < world) else (None if dp == world else None)
    # dense-gradient group: all ranks that hold the same parameter shard = same (pp, tp), any (dp, cp)
    if dp * cp == world:
        st.dp_cp_group = None  # the default group
    elif dp * cp > 1:
        mine = None
        for p in range(pp):
            for t in range(tp):
                ranks = sorted(ns.get_ranks_by_coord(pp=p, tp=t))
                g = dist.new_group(ranks=ranks, backend=backend)
                if rank in ranks:
                    mine = g
        st.dp_cp_group = mine
    else:
        st.dp_cp_group = "self"
    if ep > 1:
        # consecutive ranks of the (dp, cp) plane form an expert-parallel group
        mine = None
        for p in range(pp):
            for t in range(tp):
                plane = sorted(ns.get_ranks_by_coord(pp=p, tp=t))
                for i in range(0, len(plane), ep):
                    ranks = plane[i : i + ep]
                    g = dist.new_group(ranks=ranks, backend=backend)
                    if rank in ranks:
                        mine = g
                        st.ep_rank = ranks.index(rank)
        st.ep_group = mine
        # ranks that hold the same experts (same position inside their expert-parallel group): they all-reduce the expert
        # gradients and shard the expert optimizer state
        mine = None
        for p in range(pp):
            for t in range(tp):
                plane = sorted(ns.get_ranks_by_coord(pp=p, tp=t))
                for i in range(ep):
                    ranks = plane[i::ep]
                    if len(ranks) > 1:
                        g = dist.new_group(ranks=ranks, backend=backend)
                        if rank in ranks:
                            mine = g
                    elif rank in ranks:
                        mine = "self"
        st.extras["expert_dp_group"] = mine
        st.extras["expert_dp_size"] = (dp * cp) // ep
    if pp > 1:
        # first + last stage of every pipeline: they share the tied embedding table and all-reduce its gradient
        mine = None
        for d in range(dp):
            for c_ in range(cp):
                for t in range(tp):
                    ranks = sorted({ns.get_ranks(pp=0, dp=d, cp=c_, tp=t), ns.get_ranks(pp=pp - 1, dp=d, cp=c_, tp=t)})
                    g = dist.new_group(ranks=ranks, backend=backend)
                    if rank in ranks:
                        mine = g
        st.extras["embed_group"] = mine
    if tp * pp * cp > 1 and tp * pp * cp < world:
        mine = None
        for d in range(dp):
            ranks = sorted(ns.get_ranks_by_coord(dp=d))
            g = dist.new_group(ranks=ranks, backend=backend)
            if rank in ranks:
                mine = g
        st.model_group = mine
    _STATE = st
    return st
