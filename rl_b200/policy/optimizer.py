"""Sharded AdamW over the model's flat parameter buffer (ZeRO-1/2 style, laid out for 180 GB GPUs).

Every data-parallel rank keeps the full bf16 parameters and a full gradient-accumulation buffer resident (no
parameter all-gather inside forward / backward), and owns 1/N of the optimizer state: the low 16 bits of the fp32
master weights, and the two Adam moments. One optimizer step is

    reduce-scatter(grad) -> global grad-norm / clip scale -> AdamW on the shard -> all-gather(bf16 params)

On NVLink-connected GPUs the three stages run as one fused peer-memory kernel (:mod:`rl_b200.parallel.symmetric`);
the NCCL/gloo form below is its twin and the CPU path. The reference reaches the same end state with FSDP2
reduce-scatter + ``torch.optim.AdamW`` on DTensor shards (nemo_rl/models/automodel/setup.py:481-493, :806-820) and
``clip_grad_by_total_norm_`` (nemo_rl/models/dtensor/parallelize.py:780-882).
"""

from __future__ import annotations

import importlib
import math
from typing import Any, Optional

import torch
import torch.distributed as dist

from rl_b200.models.transformer import FlatParams
from rl_b200.ops import functional as F


def _world(group) -> tuple[int, int]:
    if isinstance(group, str):  # "self": a group of one (a single data-parallel replica inside a larger job)
        return 0, 1
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(group), dist.get_world_size(group)
    return 0, 1


class ShardedAdamW:
    def __init__(self, flat: FlatParams, *, lr: float = 1e-5, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.01, max_grad_norm: Optional[float] = None, group=None,
                 master_format: str = "split16", fused_comm: Optional[Any] = None, replicate_group=None):
        """``master_format``: ``split16`` keeps bf16 + 16 low bits (exact fp32 master at 4 B/param), ``fp32`` keeps a
        separate fp32 master shard (CPU / fp32 models use this). ``replicate_group`` (hybrid sharding): ``group`` is then one
        SHARD group (e.g. the GPUs of a node) over which the optimizer state is cut, and ``replicate_group`` holds the ranks
        of the other shard groups that own the same slice: gradients are reduce-scattered inside the shard group and the
        slices all-reduced across it, so only one slice per rank crosses the slower links between shard groups."""
        self.flat = flat
        self.group = group
        self.replicate_group = replicate_group
        self.replicas_of_shard = dist.get_world_size(replicate_group) if replicate_group is not None else 1
        self.rank, self.world = _world(group)
        assert flat.padded % self.world == 0, "flat parameter buffer must split evenly over optimizer shards"
        self.shard_numel = flat.padded // self.world
        self.lo, self.hi = self.rank * self.shard_numel, (self.rank + 1) * self.shard_numel
        self.lr, self.betas, self.eps, self.weight_decay = lr, tuple(betas), eps, weight_decay
        self.max_grad_norm = max_grad_norm
        self.step_count = 0
        dev = flat.flat.device
        p_shard = flat.flat[self.lo : self.hi]
        if flat.flat.dtype != torch.bfloat16:
            master_format = "fp32"
        self.master_format = master_format
        if master_format == "split16":
            self.p_lo = torch.zeros(self.shard_numel, dtype=torch.int16, device=dev)  # bf16 value is the exact master at start
            self.p32 = None
        else:
            self.p_lo = None
            self.p32 = p_shard.float().clone()
        self.m = torch.zeros(self.shard_numel, dtype=torch.float32, device=dev)
        self.v = torch.zeros(self.shard_numel, dtype=torch.float32, device=dev)
        self.grad_shard: Optional[torch.Tensor] = None
        self._sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        self._scale = torch.ones(1, dtype=torch.float32, device=dev)
        self._norm = torch.zeros(1, dtype=torch.float32, device=dev)
        self.fused_comm = fused_comm
        self.last_grad_norm: Optional[torch.Tensor] = None
        self._replicated: list[tuple[int, int]] = []   # shard-relative ranges replicated over the tensor-parallel group
        self._replicas = 1
        self._norm_groups: list = []
        self._excluded: list[tuple[int, int]] = []

    def set_model_parallel(self, replicated_runs: list[tuple[int, int]], replicas: int, norm_groups: list,
                           excluded_runs: Optional[list[tuple[int, int]]] = None) -> None:
        """``replicated_runs``: flat ranges whose parameters every one of ``replicas`` tensor-parallel ranks holds in full
        (their squared gradient norm must count once); ``norm_groups``: process groups over which the squared norm is
        summed besides the optimizer's own (tensor / pipeline parallel)."""
        self._replicas = int(replicas)
        self._norm_groups = list(norm_groups)
        self._replicated = [(max(a, self.lo) - self.lo, min(b, self.hi) - self.lo) for a, b in replicated_runs
                            if min(b, self.hi) > max(a, self.lo)]
        # ranges whose norm another rank of a norm group already counts (second copy of a tied table)
        self._excluded = [(max(a, self.lo) - self.lo, min(b, self.hi) - self.lo) for a, b in (excluded_runs or [])
                          if min(b, self.hi) > max(a, self.lo)]

    # ------------------------------------------------------------------ step
    def zero_grad(self) -> None:
        if self.flat.grad is not None:
            self.flat.grad.zero_()
        for p in self.flat.params:
            p.grad = None

    def _reduce_scatter(self) -> torch.Tensor:
        g = self.flat.grad
        if self.world == 1:
            if self.replicas_of_shard > 1:
                dist.all_reduce(g, op=dist.ReduceOp.SUM, group=self.replicate_group)
            return g
        mine = g[self.lo : self.hi]
        if g.is_cuda:
            # in place: NCCL reduces into this rank's own slice of the buffer (recvbuff == sendbuff + rank * count), so no
            # shard-sized temporary is needed (16 GB for a 32B model at TP4 x DP2)
            dist.reduce_scatter_tensor(mine, g, op=dist.ReduceOp.SUM, group=self.group)
        else:
            dist.all_reduce(g, op=dist.ReduceOp.SUM, group=self.group)  # gloo has no reduce-scatter
        if self.replicas_of_shard > 1:      # hybrid sharding: the same slice of every shard group
            dist.all_reduce(mine, op=dist.ReduceOp.SUM, group=self.replicate_group)
        return mine

    def _all_gather(self) -> None:
        if self.world == 1:
            return
        flat = self.flat.flat
        mine = flat[self.lo : self.hi]
        if flat.is_cuda:
            dist.all_gather_into_tensor(flat, mine, group=self.group)   # in place: this rank's slice is already where it belongs
        else:
            parts = [torch.empty_like(mine) for _ in range(self.world)]
            dist.all_gather(parts, mine.contiguous(), group=self.group)
            for r, p in enumerate(parts):
                flat[r * self.shard_numel : (r + 1) * self.shard_numel].copy_(p)

    @torch.no_grad()
    def reduce_and_sumsq(self) -> torch.Tensor:
        """First half of a step: reduce-scatter the gradients and return this optimizer's squared gradient norm, already
        summed over its own group and its model-parallel groups (a 1-element tensor). Used when several optimizers
        (dense + expert parameters) must share one clipping coefficient."""
        self.flat.fold_autograd_grads()
        self.step_count += 1
        gs = self._reduce_scatter()
        self._gs = gs
        self._sumsq.zero_()
        F.sumsq_(gs, self._sumsq)
        if self._replicas > 1 and self._replicated:
            rep = torch.zeros_like(self._sumsq)
            for a, b in self._replicated:
                F.sumsq_(gs[a:b], rep)
            self._sumsq.sub_(rep * (1.0 - 1.0 / self._replicas))
        if self._excluded:
            exc = torch.zeros_like(self._sumsq)
            for a, b in self._excluded:
                F.sumsq_(gs[a:b], exc)
            self._sumsq.sub_(exc * (1.0 / self._replicas if any(a <= x < b for x, _ in self._excluded for a, b in self._replicated) else 1.0))
        if self.world > 1:
            dist.all_reduce(self._sumsq, op=dist.ReduceOp.SUM, group=self.group)
        for g in self._norm_groups:
            dist.all_reduce(self._sumsq, op=dist.ReduceOp.SUM, group=g)
        return self._sumsq

    @torch.no_grad()
    def apply(self, total_sumsq: torch.Tensor, grad_div: float = 1.0) -> torch.Tensor:
        """Second half: clip with the (global) squared norm, AdamW on the shard, all-gather the parameters."""
        gs = self._gs
        self._gs = None
        if total_sumsq is not self._sumsq:
            self._sumsq.copy_(total_sumsq)
        if grad_div != 1.0:
            self._sumsq.mul_(1.0 / (grad_div * grad_div))
        F.clip_scale(self._sumsq, float(self.max_grad_norm or 0.0), 1.0 / grad_div, self._scale, self._norm)
        p_shard = self.flat.flat[self.lo : self.hi]
        F.adamw_step(p_shard if p_shard.dtype == torch.bfloat16 else None, self.p_lo, self.p32, gs, self.m, self.v,
                     lr=self.lr, beta1=self.betas[0], beta2=self.betas[1], eps=self.eps, weight_decay=self.weight_decay,
                     step=self.step_count, grad_scale=self._scale)
        if self.p32 is not None and p_shard.dtype != torch.bfloat16:
            p_shard.copy_(self.p32.to(p_shard.dtype))
        self._all_gather()
        self.last_grad_norm = self._norm.clone()
        return self.last_grad_norm

    @torch.no_grad()
    def step(self, grad_div: float = 1.0) -> torch.Tensor:
        """Applies one update. ``grad_div`` divides the summed gradient (1 when the loss is already normalised by
        the global token count). Returns the global gradient norm (a 1-element tensor, no host sync)."""
        if self.fused_comm is not None and self.world > 1 and self.fused_comm.usable(self):
            self.flat.fold_autograd_grads()
            self.step_count += 1
            return self.fused_comm.step(self, grad_div)
        return self.apply(self.reduce_and_sumsq(), grad_div)

    # ------------------------------------------------------------------ state
    def state_dict(self) -> dict:
        return {"step": self.step_count, "m": self.m, "v": self.v, "p_lo": self.p_lo, "p32": self.p32,
                "rank": self.rank, "world": self.world, "lr": self.lr, "master_format": self.master_format}

    def load_state_dict(self, sd: dict) -> None:
        assert sd["world"] == self.world and sd["rank"] == self.rank, "optimizer shards are tied to the data-parallel layout"
        self.step_count = int(sd["step"])
        self.m.copy_(sd["m"])
        self.v.copy_(sd["v"])
        if self.p_lo is not None and sd.get("p_lo") is not None:
            self.p_lo.copy_(sd["p_lo"])
        if self.p32 is not None and sd.get("p32") is not None:
            self.p32.copy_(sd["p32"])

    def offload_state(self) -> None:
        """Moves the moments (and master remainder) to pinned host memory (``offload_optimizer_for_logprob``)."""
        for k in ("m", "v", "p_lo", "p32"):
            t = getattr(self, k)
            if t is not None and t.is_cuda:
                setattr(self, k, t.to("cpu", non_blocking=False).pin_memory())
        torch.cuda.empty_cache()

    def reload_state(self, device) -> None:
        for k in ("m", "v", "p_lo", "p32"):
            t = getattr(self, k)
            if t is not None and not t.is_cuda and torch.device(device).type == "cuda":
                setattr(self, k, t.to(device, non_blocking=True))


# ---------------------------------------------------------------------- config glue
def build_optimizer(flat: FlatParams, policy_cfg: dict, group=None, fused_comm=None, replicate_group=None) -> ShardedAdamW:
    """Reads ``policy.optimizer = {name: <dotted class path>, kwargs: {...}}``. Adam / AdamW (any module path) map to
    the sharded fused implementation."""
    ocfg = policy_cfg.get("optimizer") or {}
    name = str(ocfg.get("name", "torch.optim.AdamW"))
    kw = dict(ocfg.get("kwargs") or {})
    short = name.rsplit(".", 1)[-1].lower()
    if short not in ("adamw", "adam", "fusedadam"):
        raise ValueError(f"optimizer '{name}' is not supported (AdamW / Adam)")
    wd = kw.get("weight_decay", 0.01 if short == "adamw" else 0.0)
    return ShardedAdamW(flat, lr=float(kw.get("lr", 1e-5)), betas=tuple(kw.get("betas", (0.9, 0.999))),
                        eps=float(kw.get("eps", 1e-8)), weight_decay=float(wd),
                        max_grad_norm=policy_cfg.get("max_grad_norm"), group=group, fused_comm=fused_comm,
                        master_format=policy_cfg.get("master_weight_format", "split16"), replicate_group=replicate_group)


class LRSchedule:
    """``policy.scheduler`` is a list of ``{name, kwargs}`` torch scheduler specs, optionally ending with
    ``{milestones: [...]}`` that chains them as a SequentialLR (nemo_rl/models/automodel/setup.py:844). The schedule is
    evaluated on a one-parameter stand-in optimizer and its learning rate copied to the sharded optimizer; it advances
    once per ``train()`` call."""

    def __init__(self, opt: ShardedAdamW, spec):
        self.opt = opt
        self._dummy = torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=opt.lr)
        self.sched = None
        if spec:
            if isinstance(spec, dict):
                spec = [spec]
            scheds, milestones = [], None
            for s in spec:
                if "milestones" in s and "name" not in s:
                    milestones = s["milestones"]
                    continue
                mod, cls = s["name"].rsplit(".", 1) if "." in s["name"] else ("torch.optim.lr_scheduler", s["name"])
                klass = getattr(importlib.import_module(mod), cls)
                scheds.append(klass(self._dummy, **(s.get("kwargs") or {})))
            if len(scheds) == 1:
                self.sched = scheds[0]
            elif scheds:
                self.sched = torch.optim.lr_scheduler.SequentialLR(self._dummy, scheds, milestones or [])
        self.opt.lr = self._dummy.param_groups[0]["lr"]

    def step(self) -> float:
        if self.sched is not None:
            self._dummy.step()
            self.sched.step()
            self.opt.lr = self._dummy.param_groups[0]["lr"]
        return self.opt.lr

    def state_dict(self):
        return {"sched": self.sched.state_dict() if self.sched is not None else None, "lr": self.opt.lr}

    def load_state_dict(self, sd):
        if self.sched is not None and sd.get("sched") is not None:
            self.sched.load_state_dict(sd["sched"])
        self.opt.lr = sd.get("lr", self.opt.lr)
        self._dummy.param_groups[0]["lr"] = self.opt.lr
