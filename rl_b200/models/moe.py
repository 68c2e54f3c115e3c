"""Mixture-of-experts feed-forward block: Qwen3-MoE style (softmax router, top-k, optional renormalisation) and DeepSeek-V3
style (sigmoid scores, a per-expert selection bias, group-limited top-k, a scaling factor, shared experts).

Tokens are sorted by expert once, each expert's SwiGLU MLP runs over its contiguous slice, and the weighted
outputs are scattered back. With expert parallelism (``ep_group``) the sorted slices are exchanged with an
all-to-all so that every rank computes only its local experts (the dispatch / combine step that the reference
delegates to mcore's token dispatchers and DeepEP, nemo_rl/models/megatron/setup.py:888-1023).
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from rl_b200.ops import functional as F

from .config import ModelConfig


class MoEMLP(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device, ep=None):
        super().__init__()
        from rl_b200.parallel.expert import EP

        self.cfg = cfg
        self.ep = ep or EP()
        ep_rank, ep_size = self.ep.rank, self.ep.world
        d, f, E = cfg.hidden_size, cfg.moe_intermediate_size, cfg.num_experts
        assert E % ep_size == 0
        self.ep_rank, self.ep_size = ep_rank, ep_size
        self.local_experts = E // ep_size
        self.router = nn.Parameter(torch.empty(E, d, dtype=dtype, device=device))
        self.gated = cfg.mlp_gated
        # Nemotron-H: the routed experts may work in a narrower ("latent") space between two shared projections
        din = cfg.moe_latent_size or d
        self.fc1_latent_proj = self.fc2_latent_proj = None
        if cfg.moe_latent_size:
            self.fc1_latent_proj = nn.Parameter(torch.empty(din, d, dtype=dtype, device=device))
            self.fc2_latent_proj = nn.Parameter(torch.empty(d, din, dtype=dtype, device=device))
        if self.gated:
            self.gate_up_proj = nn.Parameter(torch.empty(self.local_experts, 2 * f, din, dtype=dtype, device=device))
        else:   # down(act(up(x))) experts
            self.up_proj = nn.Parameter(torch.empty(self.local_experts, f, din, dtype=dtype, device=device))
        self.down_proj = nn.Parameter(torch.empty(self.local_experts, din, f, dtype=dtype, device=device))
        if cfg.scoring_func == "sigmoid":
            # selection bias of the auxiliary-loss-free load balancing: shifts which experts are chosen, never the weights;
            # not trained by gradient (a buffer, stored in checkpoints as mlp.gate.e_score_correction_bias)
            self.register_buffer("e_score_correction_bias", torch.zeros(E, dtype=torch.float32, device=device))
        self.shared_experts = None
        if cfg.n_shared_experts:
            from .transformer import DenseMLP

            self.shared_experts = DenseMLP(cfg, dtype, device, intermediate_size=cfg.moe_shared_expert_intermediate_size
                                           or cfg.moe_intermediate_size * cfg.n_shared_experts)
        self.last_routing: Optional[torch.Tensor] = None  # top-k expert ids of the last forward (router replay / traces)
        self.forced_routing: Optional[torch.Tensor] = None  # when set, replaces the router's choice (router replay); rows of -1 keep it
        self.routing_sink = None   # optional callable(layer, idx [T, k]) told every routing decision (the engine records them)

    def _route_sigmoid(self, x: torch.Tensor):
        """DeepSeek-V3 routing: sigmoid scores; experts are chosen by score + bias among the ``topk_group`` best groups (a
        group's rank is the sum of its two best biased scores); the weights are the unbiased scores, renormalised and scaled."""
        c = self.cfg
        E, k = c.num_experts, c.num_experts_per_tok
        scores = torch.sigmoid(x.float() @ self.router.float().t())
        forced = self._forced_rows(x.shape[0])
        if forced is not None and bool((forced >= 0).all()):
            idx = forced
        else:
            choice = scores + self.e_score_correction_bias
            if c.n_group > 1:
                g = choice.view(-1, c.n_group, E // c.n_group)
                gs = g.topk(2, dim=-1)[0].sum(-1)
                keep = torch.zeros_like(gs).scatter_(1, gs.topk(c.topk_group, dim=-1, sorted=False)[1], 1.0)
                choice = choice.masked_fill(~keep.bool().unsqueeze(-1).expand_as(g).reshape(-1, E), 0.0)
            idx = choice.topk(k, dim=-1, sorted=False)[1]
            if forced is not None:
                idx = torch.where((forced >= 0).all(-1, keepdim=True), forced.clamp(min=0), idx)
        w = scores.gather(1, idx)
        if c.norm_topk_prob:
            w = w / (w.sum(-1, keepdim=True) + 1e-20)
        w = w * c.routed_scaling_factor
        self.last_routing = idx.detach()
        if self.routing_sink is not None:
            self.routing_sink(self, self.last_routing)
        return w, idx, scores

    def _forced_rows(self, T: int) -> Optional[torch.Tensor]:
        """The replayed expert ids for the T rows of this call (rows the trace does not cover are -1: the router decides)."""
        f = self.forced_routing
        if f is None:
            return None
        if f.shape[0] < T:
            f = torch.cat([f, f.new_full((T - f.shape[0], f.shape[1]), -1)])
        return f[:T]

    def route(self, x: torch.Tensor):
        c = self.cfg
        if c.scoring_func == "sigmoid":
            return self._route_sigmoid(x)
        logits = F.linear(x, self.router).float()
        probs = torch.softmax(logits, dim=-1)
        w, idx = torch.topk(probs, c.num_experts_per_tok, dim=-1)
        forced = self._forced_rows(x.shape[0])
        if forced is not None:
            idx = torch.where((forced >= 0).all(-1, keepdim=True), forced.clamp(min=0), idx)
            w = probs.gather(-1, idx)
        if c.norm_topk_prob:
            w = w / w.sum(-1, keepdim=True)
        self.last_routing = idx.detach()
        if self.routing_sink is not None:
            self.routing_sink(self, self.last_routing)
        return w, idx, probs

    def _experts(self, xs: torch.Tensor, counts) -> torch.Tensor:
        """xs: tokens sorted by local expert; counts[e] tokens for local expert e (tensor or list). One grouped-GEMM MLP
        over all local experts (see :mod:`rl_b200.ops.moe_ops`)."""
        from rl_b200.ops.moe_ops import grouped_expert_mlp

        if not self.gated:
            # non-gated experts: one pair of products per expert over its slice (the split sizes are read on the host)
            cl = counts.tolist() if isinstance(counts, torch.Tensor) else list(counts)
            outs, s0 = [], 0
            up, down = self.up_proj, self.down_proj
            q_up, q_down = getattr(up, "_rlb_qat", None), getattr(down, "_rlb_qat", None)
            if q_up is not None or q_down is not None:     # quantisation-aware training (rl_b200/policy/qat.py)
                from rl_b200.policy.qat import QatState

                if QatState.enabled:
                    if q_up is not None:
                        xs, up = q_up.q_input(xs), q_up.q_weight(up)
                    if q_down is not None:
                        down = q_down.q_weight(down)
                else:
                    q_down = None
            for e, n in enumerate(cl):
                if n:
                    h = F.plain_act(torch.nn.functional.linear(xs[s0 : s0 + n], up[e]), self.cfg.hidden_act)
                    outs.append(torch.nn.functional.linear(h if q_down is None else q_down.q_input(h), down[e]))
                s0 += n
            return torch.cat(outs) if outs else xs.new_zeros((0, self.down_proj.shape[1]))
        if not isinstance(counts, torch.Tensor):
            counts = torch.tensor(counts, dtype=torch.int64, device=xs.device)
        return grouped_expert_mlp(xs, counts, self.gate_up_proj, self.down_proj)

    # ---- few-token path (decode steps): fixed shapes, no host visit, capturable in a CUDA graph
    def _small_workspace(self, T: int):
        """The shared :class:`rl_b200.ops.moe_ops.SmallTokenMoE` of this model's layers, or None when the call does not
        qualify. With expert parallelism the caller must have declared (``ep.lockstep_tokens``) that every rank of the
        group runs this layer with the same token count; only the generation engine's decode steps do."""
        from rl_b200.ops import lib as _L
        from rl_b200.ops import moe_ops as M

        c = self.cfg
        if torch.is_grad_enabled() or self.forced_routing is not None or not _L.available():
            return None
        if c.scoring_func != "softmax" or self.shared_experts is not None or not self.gated or self.fc1_latent_proj is not None \
                or getattr(self.down_proj, "_rlb_qat", None) is not None or getattr(self.gate_up_proj, "_rlb_qat", None) is not None:
            return None   # the routing kernel implements the soft-max router; other routers take the general path
        W = self.ep_size
        lock = int(getattr(self.ep, "lockstep_tokens", 0) or 0)
        if W > 1 and (lock <= 0 or self.ep.comm is None):
            return None
        max_t = max(lock, int(getattr(self.ep, "lockstep_max", 0) or 0)) if W > 1 else min(256, M.SMALL_MAX_COPIES // c.num_experts_per_tok)
        if T > max_t or W * max_t * c.num_experts_per_tok > M.SMALL_MAX_COPIES or c.hidden_size % 64 or c.moe_intermediate_size % 64 \
                or self.local_experts > 256 or c.num_experts_per_tok > 16:
            return None
        # one workspace for all layers: on the expert-parallel handle they share, or per (device, shape) without one
        key = (self.router.device, c.hidden_size, c.moe_intermediate_size, c.num_experts, c.num_experts_per_tok)
        ws = getattr(self.ep, "_small_moe", None) if W > 1 else M.SMALL_WORKSPACES.get(key)
        if ws is None or ws.maxT < max_t or ws.device != self.router.device:
            if ws is not None:
                ws.close()
            ws = M.SmallTokenMoE(c.hidden_size, c.moe_intermediate_size, c.num_experts, c.num_experts_per_tok,
                                 self.ep if W > 1 else None, max_t, self.router.device)
            if W > 1:
                self.ep._small_moe = ws
            else:
                M.SMALL_WORKSPACES[key] = ws
        return ws

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        c = self.cfg
        T, d = x.shape
        k, E = c.num_experts_per_tok, c.num_experts
        if x.is_cuda and x.dtype == torch.bfloat16 and T > 0:
            ws = self._small_workspace(T)
            if ws is not None:
                out, idx = ws.forward(x, residual, self.router, self.gate_up_proj, self.down_proj, bool(c.norm_topk_prob))
                self.last_routing = idx.clone()   # the workspace's copy is overwritten by the next layer
                if self.routing_sink is not None:
                    self.routing_sink(self, self.last_routing)
                return out
        w, idx, _ = self.route(x)
        flat_e = idx.reshape(-1)
        order = torch.argsort(flat_e, stable=True)
        tok = order // k
        x_in = x
        if self.fc1_latent_proj is not None:
            x = torch.nn.functional.linear(x, self.fc1_latent_proj)
        xs = x[tok]
        counts = torch.zeros(E, dtype=torch.int64, device=x.device).scatter_add_(0, flat_e, torch.ones_like(flat_e))
        if self.ep_size > 1:
            from rl_b200.parallel.expert import all_to_all_tokens, fused_dispatch_experts_combine

            if self.gated and getattr(self.down_proj, "_rlb_qat", None) is None and getattr(self.gate_up_proj, "_rlb_qat", None) is None \
                    and self.ep.comm is not None and xs.is_cuda and xs.dtype == torch.bfloat16 and xs.shape[0] <= self.ep.comm.max_copies:
                # dispatch, grouped expert MLP and combine over peer memory: no host-side split sizes, no NCCL all-to-all
                ys = fused_dispatch_experts_combine(xs, counts, self.ep, self.local_experts, self.gate_up_proj, self.down_proj)
            else:
                ys = all_to_all_tokens(xs, counts, self.ep, self.local_experts, self._experts)
        else:
            ys = self._experts(xs, counts)
        wy = ys * w.reshape(-1)[order].unsqueeze(-1).to(ys.dtype)
        if self.fc2_latent_proj is not None:   # sum in the latent space, one projection back for all experts
            lat = torch.zeros_like(x).index_add(0, tok, wy)
            out = torch.nn.functional.linear(lat, self.fc2_latent_proj)
            out = out if residual is None else out + residual
        else:
            out = torch.zeros_like(x) if residual is None else residual.clone()
            out = out.index_add(0, tok, wy)
        if self.shared_experts is not None:
            out = self.shared_experts(x_in, out)
        return out
