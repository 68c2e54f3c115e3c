"""Non-colocated operation: the ranks of one job are split into a TRAINING set and a GENERATION set.

``policy.generation.colocated.enabled: false`` (with ``colocated.resources.gpus_per_node`` = GPUs reserved for
generation, or ``grpo.async_grpo.generation_ranks``) takes the last G ranks of the job out of training: they run
generation engines only, while the first T = W - G ranks train. The reference does this split when it builds its Ray
virtual clusters (nemo_rl/algorithms/grpo.py:726, :811-913); in the one-process-per-GPU runtime it is a split of the
process groups:

  * every rank connects to ONE TCP store (the launcher's, or one hosted by rank 0);
  * the default ``torch.distributed`` group of a training rank contains the training ranks only, that of a generation
    rank the generation ranks only, so all existing data-parallel code runs unchanged inside its own set;
  * a raw "sync" communicator (NCCL on GPUs, gloo on CPU) spans training rank 0 and all generation ranks: weights travel
    over it; trajectories and control messages travel through the store.

Colocated jobs (G = 0) keep the ordinary bootstrap of ``rl_b200.distributed.launch.init_distributed``.
"""

from __future__ import annotations

import datetime
import os
import pickle
from dataclasses import dataclass
from typing import Any, Optional

import torch
import torch.distributed as dist


@dataclass
class RoleLayout:
    role: str                  # "colocated" | "train" | "generation"
    role_rank: int
    role_world: int
    global_rank: int
    global_world: int
    train_world: int
    gen_world: int
    device: torch.device
    store: Any = None          # the job-wide TCP store (None for colocated jobs)

    @property
    def is_trainer(self) -> bool:
        return self.role in ("colocated", "train")


def generation_ranks_from_config(cfg: dict, world: int) -> int:
    """How many ranks of the job only generate (0: colocated)."""
    gen = ((cfg.get("policy") or {}).get("generation") or {})
    col = gen.get("colocated") or {}
    a = ((cfg.get("grpo") or {}).get("async_grpo") or {})
    if a.get("generation_ranks"):
        g = int(a["generation_ranks"])
    elif col.get("enabled", True) is False:
        res = col.get("resources") or {}
        g = int(res.get("gpus_per_node") or 0) * int(res.get("num_nodes") or 1)
        if g <= 0:
            g = world // 2
    else:
        return 0
    if not 0 < g < world:
        raise ValueError(f"{g} generation ranks do not leave a training rank in a job of {world}")
    return g


def _job_store(rank: int, world: int, timeout_s: float):
    addr = os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    port = int(os.environ.setdefault("MASTER_PORT", "29500"))
    agent = os.environ.get("TORCHELASTIC_USE_AGENT_STORE", "False") == "True"   # torchrun hosts the store itself
    return dist.TCPStore(addr, port, world, is_master=(rank == 0 and not agent), timeout=datetime.timedelta(seconds=timeout_s),
                         wait_for_workers=False)


def init_roles(cfg: dict, backend: Optional[str] = None, timeout_s: float = 1800.0) -> RoleLayout:
    """Bootstraps the process groups of a colocated or a split job from the recipe. Collective over the whole job."""
    from rl_b200.distributed.launch import init_distributed

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    g = generation_ranks_from_config(cfg, world) if world > 1 else 0
    if g == 0:
        r, w, dev = init_distributed(backend, timeout_s)
        return RoleLayout("colocated", r, w, r, w, w, 0, dev)
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    use_cuda = torch.cuda.is_available() and backend != "gloo"
    device = torch.device("cuda", local) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(device)
    store = _job_store(rank, world, timeout_s)
    t = world - g
    role, rr, rw = ("train", rank, t) if rank < t else ("generation", rank - t, g)
    kw = dict(backend=backend or ("nccl" if use_cuda else "gloo"), rank=rr, world_size=rw, store=dist.PrefixStore(f"role_{role}/", store),
              timeout=datetime.timedelta(seconds=timeout_s))
    if use_cuda:
        kw["device_id"] = device
    dist.init_process_group(**kw)
    return RoleLayout(role, rr, rw, rank, world, t, g, device, store)


class SyncGroup:
    """Raw communicator over training rank 0 and all generation ranks (group rank 0 = the trainer). Created outside the
    default groups, straight on the job store. ``broadcast_object`` / ``broadcast_tensor`` are collective over the group."""

    def __init__(self, layout: RoleLayout, timeout_s: float = 1800.0):
        assert layout.store is not None and (layout.role == "generation" or layout.role_rank == 0)
        self.rank = 0 if layout.role == "train" else 1 + layout.role_rank
        self.world = 1 + layout.gen_world
        self.device = layout.device
        store = dist.PrefixStore("role_sync/", layout.store)
        to = datetime.timedelta(seconds=timeout_s)
        if self.device.type == "cuda":
            opts = dist.ProcessGroupNCCL.Options()
            opts._timeout = to
            self.pg = dist.ProcessGroupNCCL(store, self.rank, self.world, opts)
        else:
            self.pg = dist.ProcessGroupGloo(store, self.rank, self.world, to)

    def broadcast_tensor(self, t: torch.Tensor, src: int = 0) -> torch.Tensor:
        opts = dist.BroadcastOptions()
        opts.rootRank = src
        opts.rootTensor = 0
        self.pg.broadcast([t], opts).wait()
        return t

    def broadcast_object(self, obj: Any = None, src: int = 0) -> Any:
        if self.rank == src:
            payload = torch.frombuffer(bytearray(pickle.dumps(obj)), dtype=torch.uint8).to(self.device)
            n = torch.tensor([payload.numel()], dtype=torch.int64, device=self.device)
        else:
            n = torch.zeros(1, dtype=torch.int64, device=self.device)
        self.broadcast_tensor(n, src)
        if self.rank != src:
            payload = torch.empty(int(n.item()), dtype=torch.uint8, device=self.device)
        self.broadcast_tensor(payload, src)
        return obj if self.rank == src else pickle.loads(payload.cpu().numpy().tobytes())


_CURRENT: Optional[RoleLayout] = None


def set_current_layout(layout: RoleLayout) -> None:
    global _CURRENT
    _CURRENT = layout


def current_layout() -> Optional[RoleLayout]:
    """The layout the entry point bootstrapped (None when the process groups were made some other way)."""
    return _CURRENT
