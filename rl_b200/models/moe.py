"""Mixture-of-experts feed-forward block (Qwen3-MoE style: softmax router, top-k, optional renormalisation).

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
        self.gate_up_proj = nn.Parameter(torch.empty(self.local_experts, 2 * f, d, dtype=dtype, device=device))
        self.down_proj = nn.Parameter(torch.empty(self.local_experts, d, f, dtype=dtype, device=device))
        self.last_routing: Optional[torch.Tensor] = None  # top-k expert ids of the last forward (router replay / traces)
        self.forced_routing: Optional[torch.Tensor] = None  # when set, replaces the router's choice (router replay)

    def route(self, x: torch.Tensor):
        c = self.cfg
        logits = F.linear(x, self.router).float()
        probs = torch.softmax(logits, dim=-1)
        if self.forced_routing is not None:
            idx = self.forced_routing
            w = probs.gather(-1, idx)
        else:
            w, idx = torch.topk(probs, c.num_experts_per_tok, dim=-1)
        if c.norm_topk_prob:
            w = w / w.sum(-1, keepdim=True)
        self.last_routing = idx.detach()
        return w, idx, probs

    def _experts(self, xs: torch.Tensor, counts) -> torch.Tensor:
        """xs: tokens sorted by local expert; counts[e] tokens for local expert e (tensor or list). One grouped-GEMM MLP
        over all local experts (see :mod:`rl_b200.ops.moe_ops`)."""
        from rl_b200.ops.moe_ops import grouped_expert_mlp

        if not isinstance(counts, torch.Tensor):
            counts = torch.tensor(counts, dtype=torch.int64, device=xs.device)
        return grouped_expert_mlp(xs, counts, self.gate_up_proj, self.down_proj)

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        c = self.cfg
        T, d = x.shape
        k, E = c.num_experts_per_tok, c.num_experts
        w, idx, _ = self.route(x)
        flat_e = idx.reshape(-1)
        order = torch.argsort(flat_e, stable=True)
        tok = order // k
        xs = x[tok]
        counts = torch.zeros(E, dtype=torch.int64, device=x.device).scatter_add_(0, flat_e, torch.ones_like(flat_e))
        if self.ep_size > 1:
            from rl_b200.parallel.expert import all_to_all_tokens, fused_dispatch_experts_combine

            if self.ep.comm is not None and xs.is_cuda and xs.dtype == torch.bfloat16 and xs.shape[0] <= self.ep.comm.max_copies:
                # dispatch, grouped expert MLP and combine over peer memory: no host-side split sizes, no NCCL all-to-all
                ys = fused_dispatch_experts_combine(xs, counts, self.ep, self.local_experts, self.gate_up_proj, self.down_proj)
            else:
                ys = all_to_all_tokens(xs, counts, self.ep, self.local_experts, self._experts)
        else:
            ys = self._experts(xs, counts)
        wy = ys * w.reshape(-1)[order].unsqueeze(-1).to(ys.dtype)
        out = torch.zeros_like(x) if residual is None else residual.clone()
        out = out.index_add(0, tok, wy)
        return out
