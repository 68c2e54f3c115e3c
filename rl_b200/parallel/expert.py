"""Expert parallelism: token dispatch / combine between the ranks that share a MoE layer's experts.

Every rank routes its own tokens, sorts them by (global) expert, and sends each slice to the rank that owns the expert;
the owner runs its local experts over everything it received and sends the results back the same way. ``EP`` holds the
group; ``all_to_all_tokens`` is the differentiable dispatch -> experts -> combine round trip. The collective twin is
``torch.distributed.all_to_all_single`` (NCCL / gloo); on NVLink-connected GPUs the dispatch and combine copies go
through peer memory (rl_b200/csrc/moe_dispatch.cu) when an ``EPFusedComm`` is attached.

The reference delegates this step to Megatron's token dispatchers (allgather / alltoall / DeepEP flex,
nemo_rl/models/megatron/setup.py:888-1023; policy config ``moe_token_dispatcher_type``).
"""

from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist


class EP:
    def __init__(self, group=None, rank: int = 0, world: int = 1, comm=None):
        self.group, self.rank, self.world, self.comm = group, rank, world, comm

    @classmethod
    def from_state(cls, st=None) -> "EP":
        from rl_b200.parallel.state import get_state

        st = st or get_state()
        return cls(st.ep_group, st.ep_rank, st.ep, st.ep_comm)


class _AllToAllRows(torch.autograd.Function):
    """Rows of ``x`` are split by ``send`` (rows per destination) and received as ``recv`` (rows per source)."""

    @staticmethod
    def forward(ctx, x, send: list[int], recv: list[int], group):
        ctx.send, ctx.recv, ctx.group = send, recv, group
        out = torch.empty((sum(recv), *x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=recv, input_split_sizes=send, group=group)
        return out

    @staticmethod
    def backward(ctx, dy):
        dx = torch.empty((sum(ctx.send), *dy.shape[1:]), dtype=dy.dtype, device=dy.device)
        dist.all_to_all_single(dx, dy.contiguous(), output_split_sizes=ctx.send, input_split_sizes=ctx.recv, group=ctx.group)
        return dx, None, None, None


def exchange_counts(counts: torch.Tensor, ep: EP, local_experts: int) -> torch.Tensor:
    """``counts`` [E] tokens this rank sends to every global expert -> [ep, local_experts]: tokens each source rank sends
    to each of this rank's experts."""
    send = counts.view(ep.world, local_experts).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=ep.group)
    return recv


def all_to_all_tokens(xs: torch.Tensor, counts: torch.Tensor, ep: EP, local_experts: int,
                      expert_fn: Callable[[torch.Tensor, list[int]], torch.Tensor]) -> torch.Tensor:
    """``xs`` [n, d]: this rank's routed token copies sorted by global expert id, ``counts`` [E] their histogram.
    Returns the expert outputs in the same order as ``xs``."""
    recv_counts = exchange_counts(counts, ep, local_experts)            # [ep, local_experts]
    send_rows = counts.view(ep.world, local_experts).sum(1).tolist()
    rc = recv_counts.tolist()                                            # host sync: split sizes are data dependent
    recv_rows = [sum(r) for r in rc]
    got = _AllToAllRows.apply(xs, send_rows, recv_rows, ep.group)        # ordered by (source rank, local expert)
    # regroup by local expert so that each expert sees one contiguous slice
    n = got.shape[0]
    seg_start, off = [], 0
    for r in range(ep.world):
        for e in range(local_experts):
            seg_start.append((e, r, off, rc[r][e]))
            off += rc[r][e]
    order = []
    for e in range(local_experts):
        for (ee, r, o, c) in seg_start:
            if ee == e and c:
                order.append(torch.arange(o, o + c, device=xs.device))
    perm = torch.cat(order) if order else torch.empty(0, dtype=torch.long, device=xs.device)
    per_expert = [sum(rc[r][e] for r in range(ep.world)) for e in range(local_experts)]
    ys = expert_fn(got[perm] if n else got, per_expert)
    back = torch.empty_like(ys)
    if n:
        back[perm] = ys
    return _AllToAllRows.apply(back, recv_rows, send_rows, ep.group)
