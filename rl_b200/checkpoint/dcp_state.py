"""torch-DCP checkpoints with one entry per HF parameter, readable at any world size.

On disk the layout is the one ``torch.distributed.checkpoint`` produces for the reference's ``ModelState`` /
``OptimizerState`` wrappers (nemo_rl/utils/native_checkpoint.py:68-238):

    weights/    model.<hf parameter name>                         the parameter, rows sharded over the saving ranks
    optimizer/  optim.optim.state.<hf parameter name>.exp_avg     AdamW first moment (fp32)
                optim.optim.state.<hf parameter name>.exp_avg_sq  second moment (fp32)
                optim.optim.state.<hf parameter name>.step        step count (fp32 scalar)
                optim.optim.param_groups                          hyper-parameters
                optim.sched                                       scheduler state (when there is one)
                optim.optim.state.<name>.master_lo                this framework only: low 16 bits of the fp32 master

so a checkpoint written by the reference's DTensor worker loads here (``master_lo`` is then zero: the bf16 weight is
the master), and a checkpoint written here at N ranks loads at any other N: every rank saves / loads row slices
(``Shard(0)`` DTensors over a 1-D mesh) and DCP re-chunks them on load.

How the flat, fused layout of this framework maps onto per-parameter names: the optimizer keeps its moments as a
shard of one flat buffer in the *local* parameter layout (fused qkv, fused gate_up). For a save the shards are
gathered into a full flat buffer, every parameter's ``.data`` is pointed at its view of that buffer for a moment, and
the HF-name iterator of ``rl_b200/models/hf_io.py`` then yields the moments under HF names exactly as it yields the
weights. Loading runs the same steps backwards.
"""

from __future__ import annotations

import contextlib
import os
from typing import Callable, Iterator, Optional

import torch
import torch.distributed as dist


# ------------------------------------------------------------------------------------------------ helpers
def _dp(worker):
    group = getattr(worker, "dp_group", None)
    if dist.is_available() and dist.is_initialized() and worker.world > 1:
        return dist.get_rank(group), dist.get_world_size(group), group
    return 0, 1, None


def _mesh(worker):
    """1-D device mesh over the data-parallel ranks (None for a single rank)."""
    rank, world, group = _dp(worker)
    if world == 1:
        return None
    from torch.distributed.device_mesh import DeviceMesh

    dev = "cuda" if worker.device.type == "cuda" else "cpu"
    ranks = dist.get_process_group_ranks(group) if group is not None else list(range(world))
    return DeviceMesh.from_group(group if group is not None else dist.group.WORLD, dev, mesh=torch.tensor(ranks))


def _row_slice(n_rows: int, rank: int, world: int) -> tuple[int, int]:
    per = -(-n_rows // world)
    lo = min(rank * per, n_rows)
    return lo, min(lo + per, n_rows)


def _as_sharded(full: torch.Tensor, mesh, rank: int, world: int):
    """This rank's ``Shard(0)`` piece of ``full`` as a DTensor (no communication); plain tensor for one rank or 0-d."""
    if mesh is None or full.dim() == 0:
        return full.detach().clone()
    from torch.distributed.tensor import DTensor, Shard

    lo, hi = _row_slice(full.shape[0], rank, world)
    local = full[lo:hi].detach().clone().contiguous()
    return DTensor.from_local(local, mesh, [Shard(0)], run_check=False, shape=full.shape, stride=full.contiguous().stride())


def _empty_sharded(shape, dtype, device, mesh, rank: int, world: int):
    if mesh is None or len(shape) == 0:
        return torch.zeros(shape, dtype=dtype, device=device)
    from torch.distributed.tensor import DTensor, Shard

    lo, hi = _row_slice(shape[0], rank, world)
    local = torch.zeros((hi - lo, *shape[1:]), dtype=dtype, device=device)
    stride = torch.empty(shape, device="meta").stride()
    return DTensor.from_local(local, mesh, [Shard(0)], run_check=False, shape=torch.Size(shape), stride=stride)


def _full(t) -> torch.Tensor:
    return t.full_tensor() if hasattr(t, "full_tensor") else t


@contextlib.contextmanager
def _params_on(flat_params, buffer: torch.Tensor):
    """Points every parameter of ``flat_params`` at its view of ``buffer`` (same flat layout, any dtype)."""
    saved = [p.data for p in flat_params.params]
    try:
        for p, o, n, s in zip(flat_params.params, flat_params.offsets, flat_params.numels, flat_params.shapes):
            p.data = buffer[o : o + n].view(s)
        yield
    finally:
        for p, d in zip(flat_params.params, saved):
            p.data = d


def _gather_flat(shard: torch.Tensor, padded: int, worker) -> torch.Tensor:
    """All optimizer shards of one state in flat order: [padded] on the shard's device."""
    rank, world, group = _dp(worker)
    if world == 1:
        return shard
    full = torch.empty(padded, dtype=shard.dtype, device=shard.device)
    if shard.is_cuda:
        dist.all_gather_into_tensor(full, shard.contiguous(), group=group)
    else:
        dist.all_gather(list(full.chunk(world)), shard.contiguous(), group=group)
    return full


def _hf_named(worker, flat_buffer: torch.Tensor) -> Iterator[tuple[str, torch.Tensor]]:
    from rl_b200.models.hf_io import iter_hf_tensors

    with _params_on(worker.flat, flat_buffer):
        for name, t in iter_hf_tensors(worker.model):
            yield name, t


def _dcp_kwargs(worker) -> dict:
    return {} if _dp(worker)[1] > 1 else {"no_dist": True}


# ------------------------------------------------------------------------------------------------ weights
def save_model(worker, path: str) -> None:
    """``weights/``: one ``model.<hf name>`` entry per parameter, row-sharded over the data-parallel ranks."""
    import torch.distributed.checkpoint as dcp

    from rl_b200.models.hf_io import iter_hf_tensors

    rank, world, _ = _dp(worker)
    mesh = _mesh(worker)
    os.makedirs(path, exist_ok=True)
    state = {"model": {name: _as_sharded(t, mesh, rank, world) for name, t in iter_hf_tensors(worker.model)}}
    dcp.save(state, checkpoint_id=path, **_dcp_kwargs(worker))
    if rank == 0:
        worker.model_cfg.save_pretrained(path)


def _saved_entries(path: str) -> dict:
    """name -> (shape, dtype) of every tensor entry of a DCP directory."""
    from torch.distributed.checkpoint import FileSystemReader
    from torch.distributed.checkpoint.metadata import TensorStorageMetadata

    md = FileSystemReader(path).read_metadata()
    return {k: (tuple(v.size), v.properties.dtype) for k, v in md.state_dict_metadata.items() if isinstance(v, TensorStorageMetadata)}


@torch.no_grad()
def load_model(worker, path: str, strict: bool = True) -> None:
    """Loads ``model.<hf name>`` entries written at any world size (by this framework or by the reference's worker)."""
    import torch.distributed.checkpoint as dcp

    from rl_b200.models.hf_io import iter_hf_tensors, load_hf_tensors

    rank, world, _ = _dp(worker)
    mesh = _mesh(worker)
    saved = _saved_entries(path)
    want = {}
    for name, t in iter_hf_tensors(worker.model):
        key = f"model.{name}"
        if key not in saved:
            if strict:
                raise KeyError(f"{key} is not in the checkpoint at {path}")
            continue
        shape, dtype = saved[key]
        if tuple(shape) != tuple(t.shape):
            raise ValueError(f"{key}: checkpoint shape {tuple(shape)} != model shape {tuple(t.shape)}")
        want[name] = _empty_sharded(shape, dtype, worker.device, mesh, rank, world)
    state = {"model": want}
    dcp.load(state, checkpoint_id=path, **_dcp_kwargs(worker))
    load_hf_tensors(worker.model, lambda n: _full(want[n]) if n in want else None, strict=strict)


# ------------------------------------------------------------------------------------------------ optimizer
def save_optimizer(worker, path: str) -> None:
    """``optimizer/``: AdamW moments per HF parameter name (+ the master remainder), scheduler and hyper-parameters."""
    import torch.distributed.checkpoint as dcp

    opt = worker.optimizer
    rank, world, _ = _dp(worker)
    mesh = _mesh(worker)
    os.makedirs(path, exist_ok=True)
    padded = worker.flat.padded
    states: dict[str, dict] = {}
    fields = [("exp_avg", opt.m), ("exp_avg_sq", opt.v)]
    if opt.p_lo is not None:
        fields.append(("master_lo", opt.p_lo))
    if opt.p32 is not None:
        fields.append(("master_fp32", opt.p32))
    dev = worker.device
    for key, shard in fields:
        full = _gather_flat(shard.to(dev), padded, worker)
        for name, t in _hf_named(worker, full):
            states.setdefault(name, {})[key] = _as_sharded(t, mesh, rank, world)
        del full
    step = torch.tensor(float(opt.step_count))
    for name in states:
        states[name]["step"] = step.clone()
    names = list(states)
    optim = {"state": states,
             "param_groups": [dict(lr=opt.lr, betas=tuple(opt.betas), eps=opt.eps, weight_decay=opt.weight_decay, params=names)]}
    payload = {"optim": optim}
    if worker.scheduler is not None:
        payload["sched"] = worker.scheduler.state_dict()
    dcp.save({"optim": payload}, checkpoint_id=path, **_dcp_kwargs(worker))


@torch.no_grad()
def load_optimizer(worker, path: str) -> None:
    import torch.distributed.checkpoint as dcp

    opt = worker.optimizer
    rank, world, group = _dp(worker)
    mesh = _mesh(worker)
    saved = _saved_entries(path)
    dev = worker.device
    padded = worker.flat.padded
    fields = [("exp_avg", "m", torch.float32), ("exp_avg_sq", "v", torch.float32)]
    if opt.p_lo is not None:
        fields.append(("master_lo", "p_lo", torch.int16))
    if opt.p32 is not None:
        fields.append(("master_fp32", "p32", torch.float32))
    step_seen: Optional[float] = None
    for key, attr, dtype in fields:
        full = torch.zeros(padded, dtype=dtype, device=dev)
        names = [n for n, _ in _hf_named(worker, full)]
        present = [n for n in names if f"optim.optim.state.{n}.{key}" in saved]
        if not present:
            if key in ("exp_avg", "exp_avg_sq"):
                raise KeyError(f"optimizer checkpoint at {path} has no '{key}' entries")
            continue   # a checkpoint without the master remainder: the bf16 weight is the master
        want = {n: {key: _empty_sharded(saved[f"optim.optim.state.{n}.{key}"][0], dtype, dev, mesh, rank, world)} for n in present}
        if step_seen is None:
            for n in present:
                if f"optim.optim.state.{n}.step" in saved:
                    want[n]["step"] = torch.zeros((), dtype=saved[f"optim.optim.state.{n}.step"][1])
                    break
        dcp.load({"optim": {"optim": {"state": want}}}, checkpoint_id=path, **_dcp_kwargs(worker))
        for n in present:
            if "step" in want[n] and step_seen is None:
                step_seen = float(want[n]["step"])
        # write every parameter's rows back into the flat layout (the parameters point at `full` while we copy)
        from rl_b200.models.hf_io import load_hf_tensors

        with _params_on(worker.flat, full):
            load_hf_tensors(worker.model, lambda n: _full(want[n][key]) if n in want else None, strict=False)
        getattr(opt, attr).copy_(full[opt.lo : opt.hi].to(getattr(opt, attr).device))
        del full, want
    if step_seen is not None:
        opt.step_count = int(step_seen)
    if worker.scheduler is not None and any(k.startswith("optim.sched") for k in _all_keys(path)):
        sd = worker.scheduler.state_dict()
        holder = {"optim": {"sched": sd}}
        try:
            dcp.load(holder, checkpoint_id=path, **_dcp_kwargs(worker))
            worker.scheduler.load_state_dict(holder["optim"]["sched"])
        except Exception:
            pass   # a scheduler of another kind (the reference's torch schedulers): keep the configured one


def _all_keys(path: str) -> list[str]:
    from torch.distributed.checkpoint import FileSystemReader

    return list(FileSystemReader(path).read_metadata().state_dict_metadata)


def is_per_parameter_checkpoint(path: str) -> bool:
    """True for a DCP directory whose entries are ``model.<name>`` / ``optim.optim.state.<name>...``."""
    if not os.path.exists(os.path.join(path, ".metadata")):
        return False
    try:
        return any(k.startswith(("model.", "optim.optim.")) for k in _all_keys(path))
    except Exception:
        return False


# ------------------------------------------------------------------------------------------------ offline conversion
def dcp_to_hf(dcp_path: str, hf_path: str, model_cfg=None) -> str:
    """Offline, single process: a ``weights/`` DCP directory (this framework's or the reference's) -> HF safetensors."""
    import torch.distributed.checkpoint as dcp

    from rl_b200.models.config import ModelConfig
    from rl_b200.models.hf_io import load_hf_tensors, save_pretrained
    from rl_b200.models.transformer import CausalLM

    saved = {k: v for k, v in _saved_entries(dcp_path).items() if k.startswith("model.")}
    if not saved:
        raise ValueError(f"{dcp_path} holds no 'model.<name>' entries")
    cfg = model_cfg or ModelConfig.from_pretrained(dcp_path)
    tensors = {k[len("model."):]: torch.zeros(shape, dtype=dtype) for k, (shape, dtype) in saved.items()}
    dcp.load({"model": tensors}, checkpoint_id=dcp_path, no_dist=True)
    dtype = next(iter(tensors.values())).dtype
    model = CausalLM(cfg, dtype=dtype if dtype.is_floating_point else torch.bfloat16, device="cpu", init=False)
    with torch.no_grad():
        load_hf_tensors(model, tensors.get, strict=True)
    save_pretrained(model, hf_path)
    return hf_path
