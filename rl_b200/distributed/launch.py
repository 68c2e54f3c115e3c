"""Process-group bootstrap for the SPMD runtime: one process per GPU started by ``torchrun`` (or a single process).

``init_distributed()`` reads RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT, binds the process to its GPU
(and, when libnuma is present, to the GPU's NUMA node), and creates the default process group: NCCL on GPUs, gloo on
CPU. It replaces the Ray virtual cluster + worker-group construction of the reference
(nemo_rl/distributed/virtual_cluster.py:751, worker_groups.py:324-690) for single-node jobs.
"""

from __future__ import annotations

import datetime
import os
from typing import Optional

import torch
import torch.distributed as dist


def init_distributed(backend: Optional[str] = None, timeout_s: float = 1800.0, bind_numa: bool = True) -> tuple[int, int, torch.device]:
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    use_cuda = torch.cuda.is_available() and backend != "gloo"
    device = torch.device("cuda", local) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(device)
        if bind_numa:
            try:
                from rl_b200.distributed.numa import bind_to_gpu_numa_node

                bind_to_gpu_numa_node(local)
            except Exception:
                pass
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        kw = dict(backend=backend or ("nccl" if use_cuda else "gloo"), rank=rank, world_size=world,
                  timeout=datetime.timedelta(seconds=timeout_s))
        if use_cuda:
            kw["device_id"] = device
        dist.init_process_group(**kw)
    return rank, world, device


def shutdown_distributed() -> None:
    if dist.is_available() and dist.is_initialized():
        try:
            dist.barrier()
        except Exception:
            pass
        dist.destroy_process_group()
