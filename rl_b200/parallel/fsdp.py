"""Fully sharded parameters (ZeRO-3 / FSDP2 semantics) for data-parallel training of models that do not fit replicated.

``policy.parallel.data_parallel_sharding: full`` (or ``dtensor_cfg.data_parallel_sharding``). The model is cut into
UNITS (the embedding, every decoder layer, the final norm + output head). Every rank keeps 1 / dp of every unit's
parameters (bf16 or fp32), the matching slice of the fp32 gradient accumulator and of the AdamW state. A unit's full
parameters exist only while the unit computes:

  forward   gather unit u into one of two unit buffers (unit u + 1 is already being gathered into the other one on a side
            stream), point the unit's parameters at the buffer, run it WITHOUT saving activations, keep only its input;
  backward  gather the unit again (u - 1 prefetching), recompute it with autograd on, back-propagate (weight gradients
            accumulate into a unit-sized fp32 staging buffer), reduce-scatter the staging buffer into every rank's
            gradient slice, release the buffers.

So activation recomputation per unit is part of the scheme (the reference pairs ``fully_shard`` per layer with activation
checkpointing the same way for models of this size: nemo_rl/models/dtensor/parallelize.py:745-768, mixed-precision policy
nemo_rl/models/automodel/setup.py:481-493). On GPUs of one node whose shards live in peer-mapped memory the gather is a
small PULL kernel over NVLink (``rlb_p2p_pull``: a few CTAs copy the peers' slices straight into the unit buffer while
the tensor cores run the previous unit), and ``torch.distributed`` all-gather / reduce-scatter is the twin (NCCL, or gloo
on CPU where the oracle tests run).

Each rank's slice of a unit is contiguous, and the slices of all units are laid out unit after unit in ONE shard buffer
per rank, so the optimizer is a single fused AdamW launch over the shard, like the ZeRO-1 path.
"""

from __future__ import annotations

import contextlib
import ctypes as C
from dataclasses import dataclass, field
from typing import Callable, Optional, Sequence

import torch
import torch.distributed as dist
import torch.nn as nn

from rl_b200.ops import functional as F
from rl_b200.ops import lib as _L


@dataclass
class Unit:
    name: str
    params: list                     # [(qualified name, nn.Parameter)]
    offsets: list = field(default_factory=list)   # element offset of every parameter inside the unit
    shapes: list = field(default_factory=list)
    length: int = 0                  # padded element count (a multiple of 8 * dp)
    shard_off: int = 0               # offset of this rank's slice inside the shard buffers


def _units_of(model) -> list[Unit]:
    units = []
    if model.embed_tokens is not None:
        units.append(Unit("embed", [("embed_tokens", model.embed_tokens)]))
    for i, layer in enumerate(model.layers):
        units.append(Unit(f"layer{i}", [(f"layers.{i}.{n}", p) for n, p in layer.named_parameters()]))
    head = []
    if model.norm is not None:
        head.append(("norm", model.norm))
    if model.lm_head is not None:
        head.append(("lm_head", model.lm_head))
    if getattr(model, "score", None) is not None:
        head.append(("score", model.score))
    if head:
        units.append(Unit("head", head))
    return units


class ParamSharder:
    """Owns the parameter / gradient shards of a model and runs its units with gather-on-use."""

    def __init__(self, model, group=None, grad_dtype: torch.dtype = torch.float32, peer_pull: bool = True, wait_limit_s: float = 20.0):
        cfg = model.cfg
        if cfg.tie_word_embeddings and not cfg.value_head:
            raise NotImplementedError("fully sharded parameters with tied embeddings: untie the output head")
        ep = getattr(model, "ep", None)
        if (cfg.is_moe and ep is not None and ep.world > 1) or model.tp.world > 1 or model.pp_size > 1:
            raise NotImplementedError("fully sharded parameters cover dense data-parallel models (no tp / pp / ep)")
        self.model, self.group = model, group
        on = dist.is_available() and dist.is_initialized() and group != "self"
        self.rank = dist.get_rank(group) if on else 0
        self.world = dist.get_world_size(group) if on else 1
        p0 = next(model.parameters())
        self.device, self.dtype = p0.device, p0.dtype
        self.units = _units_of(model)
        self.index = {u.name: i for i, u in enumerate(self.units)}
        gran = 8 * self.world
        off = 0
        for u in self.units:
            o = 0
            for _, p in u.params:
                u.offsets.append(o)
                u.shapes.append(tuple(p.shape))
                o += -(-p.numel() // 8) * 8
            u.length = -(-o // gran) * gran
            u.shard_off = off
            off += u.length // self.world
        self.shard_numel = off
        self.max_unit = max(u.length for u in self.units)
        self.total_numel = sum(u.length for u in self.units)
        # ---- shards: parameters (model dtype), fp32 gradient accumulator
        self._peer = None
        if peer_pull and self.world > 1 and self.device.type == "cuda":
            try:
                from rl_b200.parallel.symmetric import SymmetricBuffer

                self._peer = SymmetricBuffer(self.shard_numel * p0.element_size(), group)
                self.p_shard = self._peer.tensor(self.dtype, self.shard_numel)
            except Exception as e:   # no peer access: NCCL all-gather is the twin
                print(f"[fsdp] peer-memory gather unavailable ({type(e).__name__}: {e}); using NCCL all-gather")
                self._peer = None
        if self._peer is None:
            self.p_shard = torch.zeros(self.shard_numel, dtype=self.dtype, device=self.device)
        self.g_shard = torch.zeros(self.shard_numel, dtype=torch.float32, device=self.device)
        self.grad_dtype = grad_dtype
        # ---- copy this rank's slice of every unit out of the freshly built model, then drop the full parameters
        with torch.no_grad():
            for u in self.units:
                full = torch.zeros(u.length, dtype=self.dtype, device=self.device)
                for (_, p), o in zip(u.params, u.offsets):
                    full[o : o + p.numel()].copy_(p.data.reshape(-1))
                s = u.length // self.world
                self.p_shard[u.shard_off : u.shard_off + s].copy_(full[self.rank * s : (self.rank + 1) * s])
                for _, p in u.params:
                    p.data = torch.empty(0, dtype=self.dtype, device=self.device)
                del full
        if self.device.type == "cuda":
            torch.cuda.empty_cache()
        self.active_shard = self.p_shard            # the reference policy swaps another shard in (use_shard)
        self._bufs = [torch.empty(self.max_unit, dtype=self.dtype, device=self.device) for _ in range(2)]
        self._gbufs = [None, None]                  # fp32 gradient staging, allocated on the first backward
        self._slot: dict[int, int] = {}             # unit index -> parameter buffer holding it
        self._ready: dict[int, object] = {}         # unit index -> event of a prefetch in flight
        self._side = torch.cuda.Stream(device=self.device) if self.device.type == "cuda" else None
        self._dummy = torch.zeros(1, device=self.device, requires_grad=True)
        self._direction = 1
        self.stats = dict(gathers=0, prefetch_hits=0, reduce_scatters=0, gather_bytes=0)
        self.wait_limit_s = wait_limit_s

    # ------------------------------------------------------------------ gather / release
    def _gather_into(self, ui: int, buf: torch.Tensor) -> None:
        u = self.units[ui]
        s = u.length // self.world
        mine = self.active_shard[u.shard_off : u.shard_off + s]
        out = buf[: u.length]
        self.stats["gathers"] += 1
        self.stats["gather_bytes"] += (self.world - 1) * s * mine.element_size()
        if self.world == 1:
            out.copy_(mine)
        elif self._peer is not None and self.active_shard is self.p_shard:
            lib = _L.lib()
            es = mine.element_size()
            if not hasattr(lib.rlb_p2p_pull, "_bound"):
                lib.rlb_p2p_pull.argtypes = [C.c_void_p, C.c_longlong, C.c_void_p, C.c_longlong, C.c_int, C.c_int, C.c_int, C.c_void_p]
                lib.rlb_p2p_pull.restype = C.c_int
                lib.rlb_p2p_pull._bound = True
            rc = lib.rlb_p2p_pull(self._peer.table, u.shard_off * es, out.data_ptr(), s * es, self.rank, self.world, 24,
                                  torch.cuda.current_stream().cuda_stream)
            _L.Counters.launches += 1
            if rc:
                raise RuntimeError(f"rlb_p2p_pull failed with code {rc}")
        elif mine.is_cuda:
            dist.all_gather_into_tensor(out, mine.contiguous(), group=self.group)
        else:
            dist.all_gather(list(out.chunk(self.world)), mine.contiguous(), group=self.group)

    def _prefetch(self, ui: int, slot: int) -> None:
        if not (0 <= ui < len(self.units)) or ui in self._slot or ui in self._ready:
            return
        if self._side is None:
            return
        # the buffer's previous user was enqueued on the compute stream before this point
        self._side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self._side):
            self._gather_into(ui, self._bufs[slot])
            ev = torch.cuda.Event()
            ev.record()
        self._ready[ui] = (slot, ev)

    def acquire(self, ui: int, backward: bool = False) -> None:
        """Makes unit ``ui``'s full parameters available (and starts gathering its successor in compute order)."""
        u = self.units[ui]
        if ui in self._ready:
            slot, ev = self._ready.pop(ui)
            torch.cuda.current_stream().wait_event(ev)
            self.stats["prefetch_hits"] += 1
        else:
            busy = set(self._slot.values()) | {s for s, _ in self._ready.values()}
            slot = 0 if 0 not in busy else 1
            if slot in busy:
                raise RuntimeError("both unit buffers are in use: release a unit before acquiring another")
            self._gather_into(ui, self._bufs[slot])
        self._slot[ui] = slot
        buf = self._bufs[slot]
        for (_, p), o, shp in zip(u.params, u.offsets, u.shapes):
            n = 1
            for x in shp:
                n *= x
            p.data = buf[o : o + n].view(shp)
        if backward:
            if self._gbufs[slot] is None:
                self._gbufs[slot] = torch.zeros(self.max_unit, dtype=torch.float32, device=self.device)
            g = self._gbufs[slot]
            g[: u.length].zero_()
            for (_, p), o, shp in zip(u.params, u.offsets, u.shapes):
                n = p.numel()
                p.main_grad = g[o : o + n].view(shp)
                p.grad = None
        self._prefetch(ui + (-1 if backward else 1), 1 - slot)

    def release(self, ui: int) -> None:
        u = self.units[ui]
        self._slot.pop(ui, None)
        for _, p in u.params:
            p.data = torch.empty(0, dtype=self.dtype, device=self.device)
            if hasattr(p, "main_grad"):
                del p.main_grad
            p.grad = None

    @torch.no_grad()
    def reduce_grads(self, ui: int) -> None:
        """Sums unit ``ui``'s staged gradients over the ranks and adds this rank's slice to its gradient shard."""
        u = self.units[ui]
        slot = self._slot[ui]
        g = self._gbufs[slot]
        for _, p in u.params:          # gradients that autograd returned instead of accumulating in place
            if p.grad is not None:
                p.main_grad.add_(p.grad.to(torch.float32))
                p.grad = None
        s = u.length // self.world
        dst = self.g_shard[u.shard_off : u.shard_off + s]
        full = g[: u.length]
        self.stats["reduce_scatters"] += 1
        if self.world == 1:
            dst.add_(full)
        elif full.is_cuda:
            piece = torch.empty_like(dst)
            dist.reduce_scatter_tensor(piece, full, op=dist.ReduceOp.SUM, group=self.group)
            dst.add_(piece)
        else:
            dist.all_reduce(full, op=dist.ReduceOp.SUM, group=self.group)   # gloo has no reduce-scatter
            dst.add_(full[self.rank * s : (self.rank + 1) * s])

    # ------------------------------------------------------------------ running units
    def run(self, name: str, fn: Callable, *inputs: torch.Tensor):
        """Runs ``fn(*inputs)`` (which uses the parameters of unit ``name``) with the unit gathered. Under autograd only
        the inputs are kept and the unit is recomputed in backward."""
        ui = self.index[name]
        if torch.is_grad_enabled():
            return _UnitFn.apply(self, ui, fn, self._dummy, *inputs)
        self.acquire(ui)
        try:
            return fn(*inputs)
        finally:
            self.release(ui)

    @contextlib.contextmanager
    def use_shard(self, shard: torch.Tensor):
        """Runs the model on another parameter shard of the same layout (the reference policy)."""
        prev = self.active_shard
        self.active_shard = shard
        self._ready.clear()
        try:
            yield
        finally:
            self.active_shard = prev
            self._ready.clear()

    def zero_grad(self) -> None:
        self.g_shard.zero_()

    # ------------------------------------------------------------------ whole-model access (checkpoints, refit)
    @torch.no_grad()
    def iter_full_params(self):
        """Yields (qualified parameter name, full tensor) unit by unit; the tensor is valid until the next item."""
        for ui, u in enumerate(self.units):
            self.acquire(ui)
            try:
                for name, p in u.params:
                    yield name, p.data
            finally:
                self.release(ui)

    @torch.no_grad()
    def load_full_params(self, get: Callable[[str], Optional[torch.Tensor]]) -> None:
        """Fills the shard from full tensors by parameter name (``get`` returns None for names it does not have)."""
        for u in self.units:
            full = torch.zeros(u.length, dtype=self.dtype, device=self.device)
            s = u.length // self.world
            self._gather_units_own(u, full)
            for (name, _), o, shp in zip(u.params, u.offsets, u.shapes):
                t = get(name)
                if t is not None:
                    full[o : o + t.numel()].copy_(t.reshape(-1).to(self.dtype))
            self.p_shard[u.shard_off : u.shard_off + s].copy_(full[self.rank * s : (self.rank + 1) * s])

    def _gather_units_own(self, u: Unit, full: torch.Tensor) -> None:
        ui = self.index[u.name]
        self._gather_into(ui, full)
        if self.device.type == "cuda":
            torch.cuda.current_stream().synchronize()

    def close(self) -> None:
        if self._peer is not None:
            self.p_shard = None
            self.active_shard = None
            self._peer.close()
            self._peer = None


class _UnitFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, sharder: ParamSharder, ui: int, fn: Callable, dummy: torch.Tensor, *inputs):
        sharder.acquire(ui)
        try:
            with torch.no_grad():
                out = fn(*inputs)
        finally:
            sharder.release(ui)
        ctx.sharder, ctx.ui, ctx.fn = sharder, ui, fn
        ctx.save_for_backward(*[x for x in inputs if isinstance(x, torch.Tensor)])
        ctx.is_tensor = [isinstance(x, torch.Tensor) for x in inputs]
        ctx.others = [None if isinstance(x, torch.Tensor) else x for x in inputs]
        ctx.tuple_out = isinstance(out, tuple)
        return out

    @staticmethod
    def backward(ctx, *douts):
        sh, ui = ctx.sharder, ctx.ui
        saved = list(ctx.saved_tensors)
        inputs = []
        for is_t, other in zip(ctx.is_tensor, ctx.others):
            if is_t:
                x = saved.pop(0).detach()
                if x.is_floating_point():
                    x.requires_grad_(True)
                inputs.append(x)
            else:
                inputs.append(other)
        sh.acquire(ui, backward=True)
        try:
            with torch.enable_grad():
                out = ctx.fn(*inputs)
            outs = out if isinstance(out, tuple) else (out,)
            pairs = [(o, d) for o, d in zip(outs, douts) if isinstance(o, torch.Tensor) and o.requires_grad and d is not None]
            if pairs:
                torch.autograd.backward([o for o, _ in pairs], [d for _, d in pairs])
            sh.reduce_grads(ui)
        finally:
            sh.release(ui)
        grads = [x.grad if (isinstance(x, torch.Tensor) and x.requires_grad) else None for x in inputs]
        return (None, None, None, torch.zeros_like(sh._dummy), *grads)


class ShardOptimizer:
    """AdamW over one rank's parameter shard (the ZeRO-3 counterpart of ``ShardedAdamW``): global gradient-norm clipping,
    then one fused update of the shard; nothing is gathered afterwards, parameters stay sharded."""

    def __init__(self, sharder: ParamSharder, *, lr: float = 1e-5, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01,
                 max_grad_norm: Optional[float] = None):
        self.sh = sharder
        self.group, self.rank, self.world = sharder.group, sharder.rank, sharder.world
        self.lr, self.betas, self.eps, self.weight_decay, self.max_grad_norm = lr, tuple(betas), eps, weight_decay, max_grad_norm
        self.step_count = 0
        n, dev = sharder.shard_numel, sharder.device
        self.shard_numel, self.lo, self.hi = n, 0, n
        if sharder.dtype == torch.bfloat16:
            self.master_format = "split16"
            self.p_lo = torch.zeros(n, dtype=torch.int16, device=dev)
            self.p32 = None
        else:
            self.master_format = "fp32"
            self.p_lo = None
            self.p32 = sharder.p_shard.float().clone()
        self.m = torch.zeros(n, dtype=torch.float32, device=dev)
        self.v = torch.zeros(n, dtype=torch.float32, device=dev)
        self._sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        self._scale = torch.ones(1, dtype=torch.float32, device=dev)
        self._norm = torch.zeros(1, dtype=torch.float32, device=dev)
        self.last_grad_norm: Optional[torch.Tensor] = None

    def zero_grad(self) -> None:
        self.sh.zero_grad()

    @torch.no_grad()
    def step(self, grad_div: float = 1.0) -> torch.Tensor:
        self.step_count += 1
        gs = self.sh.g_shard
        self._sumsq.zero_()
        F.sumsq_(gs, self._sumsq)
        if self.world > 1:
            dist.all_reduce(self._sumsq, op=dist.ReduceOp.SUM, group=self.group)
        if grad_div != 1.0:
            self._sumsq.mul_(1.0 / (grad_div * grad_div))
        F.clip_scale(self._sumsq, float(self.max_grad_norm or 0.0), 1.0 / grad_div, self._scale, self._norm)
        p = self.sh.p_shard
        F.adamw_step(p if p.dtype == torch.bfloat16 else None, self.p_lo, self.p32, gs, self.m, self.v, lr=self.lr, beta1=self.betas[0],
                     beta2=self.betas[1], eps=self.eps, weight_decay=self.weight_decay, step=self.step_count, grad_scale=self._scale)
        if self.p32 is not None and p.dtype != torch.bfloat16:
            p.copy_(self.p32.to(p.dtype))
        if self.world > 1 and self.sh._peer is not None:
            dist.barrier(group=self.group)   # peers pull from this shard: nobody starts the next gather before every update landed
        self.sh._ready.clear()
        self.last_grad_norm = self._norm.clone()
        return self.last_grad_norm

    def state_dict(self) -> dict:
        return {"step": self.step_count, "m": self.m, "v": self.v, "p_lo": self.p_lo, "p32": self.p32, "rank": self.rank,
                "world": self.world, "lr": self.lr, "master_format": self.master_format, "sharding": "full"}

    def load_state_dict(self, sd: dict) -> None:
        assert sd["world"] == self.world and sd["rank"] == self.rank and sd.get("sharding") == "full", \
            "optimizer shards are tied to the layout that wrote them"
        self.step_count = int(sd["step"])
        self.m.copy_(sd["m"])
        self.v.copy_(sd["v"])
        if self.p_lo is not None and sd.get("p_lo") is not None:
            self.p_lo.copy_(sd["p_lo"])
        if self.p32 is not None and sd.get("p32") is not None:
            self.p32.copy_(sd["p32"])

    def offload_state(self) -> None:
        pass

    def reload_state(self, device) -> None:
        pass


# ------------------------------------------------------------------------------------------------ HF-named access
@torch.no_grad()
def iter_hf_tensors_sharded(model, sharder: ParamSharder):
    """(HF name, full tensor) for every tensor of a fully sharded model, gathered unit by unit. Collective over the data-
    parallel group; the yielded tensor is valid until the generator advances."""
    from rl_b200.models.hf_io import _model_map

    rows_of = {}
    for hf, loc, rows, e, hs in _model_map(model):
        rows_of.setdefault(loc, []).append((hf, rows, e))
    for ui, u in enumerate(sharder.units):
        sharder.acquire(ui)
        try:
            for name, p in u.params:
                for hf, rows, e in rows_of.pop(name, []):
                    t = p.data if e is None else p.data[e]      # (stacked experts: one HF tensor per expert)
                    yield hf, (t if rows is None else t[rows[0] : rows[1]])
        finally:
            sharder.release(ui)
    buffers = dict(model.named_buffers())
    for name, items in rows_of.items():      # stored buffers (router selection biases) are replicated, not sharded
        if name in buffers:
            for hf, rows, e in items:
                yield hf, buffers[name]


class ShardedServingSync:
    """Refit for a fully sharded trainer: every rank gets a serving copy of the weights in the engine's layout (tensor
    parallel size ``tp_serve``), rebuilt unit by unit from the gathered parameters. The copy costs ``params / tp_serve``
    bytes per rank; only one unit of full training parameters exists at any time."""

    def __init__(self, worker, tp_serve: int, serve_group=None, serve_comm=None):
        from rl_b200.models.hf_io import iter_hf_shards
        from rl_b200.refit.plan import serving_param_layout
        from rl_b200.refit.synchronizer import build_serving_model

        self.worker, self.tp_serve = worker, tp_serve
        cfg = worker.model_cfg
        p_dtype, dev = worker.sharder.dtype, worker.sharder.device
        _, numel = serving_param_layout(cfg, tp_serve)
        self.arena = torch.zeros(numel, dtype=p_dtype, device=dev)
        rank = dist.get_rank() if dist.is_initialized() else 0
        self.serving_model = build_serving_model(cfg, tp_serve, rank % tp_serve, self.arena, serve_group, serve_comm)
        self._dst = {hf: (dst, hs) for hf, dst, hs in iter_hf_shards(self.serving_model)}
        self.last_bytes = 0

    @torch.no_grad()
    def sync_weights(self, timer=None) -> None:
        total = 0
        for hf, t in iter_hf_tensors_sharded(self.worker.model, self.worker.sharder):
            hit = self._dst.get(hf)
            if hit is None:
                continue
            dst, hs = hit
            src = t if hs is None else t.narrow(hs[0], hs[1], hs[2])
            dst.copy_(src.to(dst.dtype))
            total += dst.numel() * dst.element_size()
        self.last_bytes = total

    def close(self) -> None:
        pass
