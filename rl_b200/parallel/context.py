"""Context parallelism for long sequences: the packed token stream is split into ``cp`` contiguous row ranges, every
layer except attention works on local rows only, and attention all-gathers the (GQA-small) keys and values of the whole
stream so that local queries can attend to every earlier token of their sequence ("all-gather KV" context parallelism;
gradients of K/V flow back through a reduce-scatter).

This is the functional path (PyTorch scaled-dot-product attention per sequence segment). The reference gets context
parallelism from DTensor ``context_parallel`` / Megatron ``context_parallel_size`` with ring attention
(nemo_rl/models/dtensor/parallelize.py:610-700, docs/design-docs/sequence-packing-and-dynamic-batching.md).
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from rl_b200.parallel.tensor import all_gather_rows, reduce_scatter_rows


class CP:
    def __init__(self, group=None, rank: int = 0, world: int = 1):
        self.group, self.rank, self.world = group, rank, world

    @classmethod
    def from_state(cls, st=None) -> "CP":
        from rl_b200.parallel.state import get_state

        st = st or get_state()
        return cls(st.cp_group, st.cp_rank, st.cp)

    def local_rows(self, total: int) -> tuple[int, int]:
        rows = total // self.world
        return self.rank * rows, (self.rank + 1) * rows


class _GatherRowsScatterGrad(torch.autograd.Function):
    """All-gather rows in forward; every rank's gradient of the gathered tensor is partial, so backward reduce-scatters."""

    @staticmethod
    def forward(ctx, x, cp: CP):
        ctx.cp = cp
        return all_gather_rows(x, cp.group, cp.world)

    @staticmethod
    def backward(ctx, dy):
        cp = ctx.cp
        return reduce_scatter_rows(dy.contiguous(), cp.group, cp.world, cp.rank), None


def cp_attention_varlen(qkv_local: torch.Tensor, cu_seqlens: torch.Tensor, cp: CP, hq: int, hkv: int, d: int,
                        scale: Optional[float] = None) -> torch.Tensor:
    """``qkv_local`` [T/cp, (hq + 2 hkv) d]: fused q, k, v of this rank's rows (already rotated). Returns the attention
    output of the local rows [T/cp, hq d] with causal masking inside every packed sequence."""
    rows = qkv_local.shape[0]
    r0 = cp.rank * rows
    q = qkv_local[:, : hq * d].reshape(rows, hq, d)
    kv = _GatherRowsScatterGrad.apply(qkv_local[:, hq * d :].contiguous(), cp)  # [T, 2 hkv d]
    k = kv[:, : hkv * d].reshape(-1, hkv, d)
    v = kv[:, hkv * d :].reshape(-1, hkv, d)
    scale = scale if scale is not None else d ** -0.5
    cu = cu_seqlens.tolist()
    out = torch.zeros((rows, hq, d), dtype=qkv_local.dtype, device=qkv_local.device)
    pieces = []
    rep = hq // hkv
    for s, e in zip(cu[:-1], cu[1:]):
        lo, hi = max(s, r0), min(e, r0 + rows)
        if hi <= lo:
            continue
        qs = q[lo - r0 : hi - r0].transpose(0, 1)                       # [hq, nq, d]
        ks = k[s:hi].transpose(0, 1).repeat_interleave(rep, dim=0)      # [hq, nk, d]
        vs = v[s:hi].transpose(0, 1).repeat_interleave(rep, dim=0)
        nq, nk = hi - lo, hi - s
        qi = torch.arange(lo - s, hi - s, device=q.device)[:, None]
        kj = torch.arange(nk, device=q.device)[None, :]
        mask = kj <= qi
        o = torch.nn.functional.scaled_dot_product_attention(qs.float(), ks.float(), vs.float(), attn_mask=mask, scale=scale)
        pieces.append((lo - r0, hi - r0, o.transpose(0, 1).to(qkv_local.dtype)))
    # packed sequences tile the stream, so the segments of the local range are contiguous and cover it
    out = torch.cat([p[2] for p in pieces], 0) if pieces else out
    return out.reshape(rows, hq * d)
