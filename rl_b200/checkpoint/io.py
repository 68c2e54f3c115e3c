"""Model / optimizer state on disk: HF safetensors, ``torch.save`` and torch-DCP (distributed checkpoint).

* ``safetensors`` (default): rank 0 writes the HF layout (every rank holds the full bf16 parameters), so the result
  loads in ``transformers`` and in this package alike. With expert parallelism each rank writes its own experts.
* ``torch_save``: one ``model.pt`` state dict in HF names.
* ``dcp``: ``torch.distributed.checkpoint`` with one entry per HF parameter name (``model.<name>``,
  ``optim.optim.state.<name>.exp_avg`` ...), the on-disk form of nemo_rl/utils/native_checkpoint.py:68-238: written at N
  ranks it loads at any other N, and a checkpoint of the reference's DTensor worker loads here
  (``rl_b200/checkpoint/dcp_state.py``); ``convert_dcp_to_hf`` rebuilds HF tensors from either.

Optimizer state: ``dcp`` writes per-parameter moments next to the weights; the other formats write one
``optimizer/rank_<r>.pt`` per rank (moments + master remainder), tied to the layout that wrote it.
"""

from __future__ import annotations

import json
import os
from typing import Optional

import torch
import torch.distributed as dist


def _rank_world(group=None):
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(group), dist.get_world_size(group)
    return 0, 1


def save_weights(worker, path: str, fmt: str = "safetensors") -> None:
    from rl_b200.models.hf_io import iter_hf_tensors, save_pretrained

    from rl_b200.models.hf_io import save_roles
    from rl_b200.parallel.state import get_state

    rank, world = (worker.rank, worker.world)
    fmt = (fmt or "safetensors").lower()
    st = get_state()
    if getattr(worker, "sharder", None) is not None:
        # fully sharded parameters: tensors are gathered unit by unit; rank 0 writes them out (HF safetensors)
        from rl_b200.parallel.fsdp import iter_hf_tensors_sharded

        sd = {}
        for n, t in iter_hf_tensors_sharded(worker.model, worker.sharder):
            if rank == 0:
                sd[n] = t.detach().to("cpu", copy=True)
        if rank == 0:
            from safetensors.torch import save_file

            os.makedirs(path, exist_ok=True)
            save_file(sd, os.path.join(path, "model.safetensors"), metadata={"format": "pt"})
            worker.model_cfg.save_pretrained(path)
        return
    if getattr(worker, "lora_cfg", None) is not None:
        # LoRA: the frozen base goes out as a plain HF checkpoint, the adapters next to it in the PEFT file layout
        if rank == 0:
            from rl_b200.models.hf_io import save_lora_adapter

            save_pretrained(worker.model, path)
            save_lora_adapter(worker.model, path)
        return
    if st.tp * st.pp * st.ep * st.cp > 1:
        # model-parallel layouts always write HF safetensors (one file set per pipeline stage / expert-parallel rank)
        if save_roles(st)[0]:
            save_pretrained(worker.model, path)
        return
    if fmt == "dcp":
        # one entry per HF parameter name, row-sharded over the saving ranks: loads at any world size, and in the
        # reference's DTensor worker (rl_b200/checkpoint/dcp_state.py)
        from rl_b200.checkpoint.dcp_state import save_model

        save_model(worker, path)
        return
    if rank != 0:
        return
    if fmt == "torch_save":
        os.makedirs(path, exist_ok=True)
        sd = {n: t.detach().cpu().clone() for n, t in iter_hf_tensors(worker.model)}
        torch.save(sd, os.path.join(path, "model.pt"))
        worker.model_cfg.save_pretrained(path)
    else:
        save_pretrained(worker.model, path)


@torch.no_grad()
def load_weights(worker, path: str) -> None:
    from rl_b200.models.hf_io import _SafetensorsDir, load_hf_tensors

    rank, world = (worker.rank, worker.world)
    if getattr(worker, "sharder", None) is not None:
        from rl_b200.models.hf_io import _SafetensorsDir, _model_map

        reader = _SafetensorsDir(path)
        by_param = {}
        for hf, loc, rows, e, hs in _model_map(worker.model):
            by_param.setdefault(loc, []).append((hf, rows, e))

        def rows_of(parts):   # one (expert's) matrix from its HF pieces, in row order
            if len(parts) == 1 and parts[0][1] is None:
                return reader.get(parts[0][0])
            return torch.cat([reader.get(hf) for hf, _, _ in sorted(parts, key=lambda x: x[1][0])], dim=0)

        def get(name):   # full local parameter assembled from its HF pieces (stacked experts: one matrix per expert)
            parts = by_param.get(name)
            if not parts:
                return None
            if parts[0][2] is None:
                return rows_of(parts)
            experts = sorted({e for _, _, e in parts})
            return torch.stack([rows_of([p for p in parts if p[2] == e]) for e in experts])

        worker.sharder.load_full_params(get)
        for bname, b in worker.model.named_buffers():      # stored buffers (router selection biases) are not sharded
            if bname in by_param:
                b.copy_(reader.get(by_param[bname][0][0]).to(b.dtype))
        return
    from rl_b200.checkpoint.dcp_state import is_per_parameter_checkpoint

    if is_per_parameter_checkpoint(path):
        from rl_b200.checkpoint.dcp_state import load_model

        load_model(worker, path)
        return
    if os.path.exists(os.path.join(path, "flat_layout.json")):   # flat-shard DCP of earlier versions (same world size only)
        import torch.distributed.checkpoint as dcp

        meta = json.load(open(os.path.join(path, "flat_layout.json")))
        assert meta["world"] == world, "DCP flat shards are tied to the data-parallel size they were written with"
        opt = worker.optimizer
        lo, hi = (opt.lo, opt.hi) if opt is not None else (0, worker.flat.padded)
        state = {"model": {f"flat.rank{rank}": torch.empty_like(worker.flat.flat[lo:hi])}}
        dcp.load(state, checkpoint_id=path, **({} if world > 1 else {"no_dist": True}))
        worker.flat.flat[lo:hi].copy_(state["model"][f"flat.rank{rank}"])
        if world > 1:
            dist.all_gather_into_tensor(worker.flat.flat, worker.flat.flat[lo:hi].clone(), group=worker.dp_group)
        return
    if os.path.exists(os.path.join(path, "model.pt")):
        sd = torch.load(os.path.join(path, "model.pt"), map_location="cpu")
        load_hf_tensors(worker.model, sd.get)
        return
    reader = _SafetensorsDir(path)
    load_hf_tensors(worker.model, reader.get)


def _global_rank() -> int:
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def save_optimizer_shard(worker, path: str, fmt: str = "safetensors") -> None:
    """One file per rank (named by the global rank: optimizer shards are tied to the whole parallel layout), or with
    ``fmt = "dcp"`` on a data-parallel layout a torch-DCP directory with per-parameter entries that loads at any world size."""
    from rl_b200.parallel.state import get_state

    st = get_state()
    if (fmt or "").lower() == "dcp" and st.tp * st.pp * st.ep * st.cp == 1 and getattr(worker, "lora_cfg", None) is None:
        from rl_b200.checkpoint.dcp_state import save_optimizer

        save_optimizer(worker, path)
        return
    os.makedirs(path, exist_ok=True)
    sd = {k: (v.detach().cpu() if isinstance(v, torch.Tensor) else v) for k, v in worker.optimizer.state_dict().items()}
    sd["scheduler"] = worker.scheduler.state_dict() if worker.scheduler is not None else None
    if getattr(worker, "optimizer_e", None) is not None:
        sd["experts"] = {k: (v.detach().cpu() if isinstance(v, torch.Tensor) else v) for k, v in worker.optimizer_e.state_dict().items()}
    torch.save(sd, os.path.join(path, f"rank_{_global_rank()}.pt"))


def load_optimizer_shard(worker, path: str) -> None:
    from rl_b200.checkpoint.dcp_state import is_per_parameter_checkpoint

    if is_per_parameter_checkpoint(path):
        from rl_b200.checkpoint.dcp_state import load_optimizer

        load_optimizer(worker, path)
        return
    f = os.path.join(path, f"rank_{_global_rank()}.pt")
    sd = torch.load(f, map_location=worker.device, weights_only=False)
    worker.optimizer.load_state_dict(sd)
    if getattr(worker, "optimizer_e", None) is not None and sd.get("experts") is not None:
        worker.optimizer_e.load_state_dict(sd["experts"])
    if worker.scheduler is not None and sd.get("scheduler") is not None:
        worker.scheduler.load_state_dict(sd["scheduler"])


def convert_dcp_to_hf(dcp_path: str, hf_path: str) -> str:
    """Offline: DCP flat shards -> HF safetensors directory (examples/converters/convert_dcp_to_hf.py in the reference)."""
    import torch.distributed.checkpoint as dcp

    from rl_b200.models.config import ModelConfig
    from rl_b200.models.hf_io import save_pretrained
    from rl_b200.models.transformer import CausalLM

    from rl_b200.checkpoint.dcp_state import dcp_to_hf, is_per_parameter_checkpoint

    if is_per_parameter_checkpoint(dcp_path):
        return dcp_to_hf(dcp_path, hf_path)
    meta = json.load(open(os.path.join(dcp_path, "flat_layout.json")))
    cfg = ModelConfig.from_pretrained(dcp_path)
    dtype = getattr(torch, meta["dtype"].replace("torch.", ""))
    model = CausalLM(cfg, dtype=dtype, device="cpu", init=False)
    flat = model.flatten_parameters(align=1)
    world = meta["world"]
    shard = meta["padded"] // world
    full = torch.zeros(meta["padded"], dtype=dtype)
    state = {"model": {f"flat.rank{r}": torch.empty(shard, dtype=dtype) for r in range(world)}}
    dcp.load(state, checkpoint_id=dcp_path, no_dist=True)
    for r in range(world):
        full[r * shard : (r + 1) * shard] = state["model"][f"flat.rank{r}"]
    name_to = {n: (o, k) for n, o, k in zip(meta["names"], meta["offsets"], meta["numels"])}
    with torch.no_grad():
        for n, o, k, s in flat.named_slices():
            so, sk = name_to[n]
            flat.flat[o : o + k].copy_(full[so : so + sk])
    save_pretrained(model, hf_path)
    return hf_path
