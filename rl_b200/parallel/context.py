"""Context parallelism for long sequences: ring attention over a load-balanced ("zig-zag") split of the token stream.

The packed stream of T rows is cut into 2 * cp chunks; rank r owns chunks r and 2 * cp - 1 - r, so under a causal mask
every rank has the same amount of attention work (the first chunks see little context, the last ones a lot; pairing them
evens it out; nemo_rl/distributed/model_utils.py:1199-1233 shards each sequence the same way). Everything except
attention is row-wise and runs on the local rows only.

Attention is a RING: every rank keeps its queries; the key / value blocks travel around the ring (send to rank + 1, receive
from rank - 1), one hop per step, the transfer of the next block overlapping the computation on the current one. A rank
folds each visiting block into its running result with the online-softmax recurrence (running maximum, running sum,
rescaled accumulator), so no rank ever holds the keys of the whole stream and nothing of size T x T exists. Blocks that
lie entirely in a query chunk's future are skipped. The backward pass runs the ring again: a block's key / value
gradients travel with it and arrive back at its owner after cp hops.

Causality and packing are decided per (query row, key row) from the rows' positions in the stream: visible iff both rows
belong to the same packed sequence and the key row is not after the query row.

The block computations are PyTorch matrix products on [heads, q tile, block] score tiles (fp32 on CPU, the model dtype
with fp32 soft-max statistics on GPUs): the functional form of the ring; the reference gets the same algorithm from
DTensor's ``context_parallel`` ring attention (nemo_rl/models/policy/workers/dtensor_policy_worker.py:536-560).
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


class CP:
    def __init__(self, group=None, rank: int = 0, world: int = 1):
        self.group, self.rank, self.world = group, rank, world

    @classmethod
    def from_state(cls, st=None) -> "CP":
        from rl_b200.parallel.state import get_state

        st = st or get_state()
        return cls(st.cp_group, st.cp_rank, st.cp)

    # ---- zig-zag ownership of stream rows
    def chunk_rows(self, total: int) -> int:
        assert total % (2 * self.world) == 0, f"{total} rows do not split into {2 * self.world} chunks"
        return total // (2 * self.world)

    def chunks_of(self, rank: int) -> tuple[int, int]:
        return rank, 2 * self.world - 1 - rank

    def local_index(self, total: int, device=None) -> torch.Tensor:
        """Stream rows owned by this rank, in local order (chunk ``rank`` first, then chunk ``2 cp - 1 - rank``)."""
        c = self.chunk_rows(total)
        a, b = self.chunks_of(self.rank)
        return torch.cat([torch.arange(a * c, (a + 1) * c, device=device), torch.arange(b * c, (b + 1) * c, device=device)])

    def stream_order(self, total: int, device=None) -> torch.Tensor:
        """Permutation that puts rows gathered rank by rank (each in local order) back into stream order."""
        c = self.chunk_rows(total)
        src = torch.cat([torch.cat([torch.arange(a * c, (a + 1) * c), torch.arange(b * c, (b + 1) * c)])
                         for a, b in (self.chunks_of(r) for r in range(self.world))])
        inv = torch.empty_like(src)
        inv[src] = torch.arange(total)
        return inv.to(device) if device is not None else inv

    def local_rows(self, total: int) -> tuple[int, int]:
        """Contiguous split (kept for callers that only need equal row counts)."""
        rows = total // self.world
        return self.rank * rows, (self.rank + 1) * rows


def gather_to_stream(x_local: torch.Tensor, cp: CP) -> torch.Tensor:
    """All-gathers per-row values of the local rows and returns them in stream order (differentiable: the backward of a
    replicated consumer hands every rank the gradient of its own rows)."""
    return _GatherStream.apply(x_local, cp)


class _GatherStream(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cp: CP):
        from rl_b200.parallel.tensor import all_gather_rows

        ctx.cp = cp
        full = all_gather_rows(x.contiguous(), cp.group, cp.world)
        ctx.total = full.shape[0]
        return full[cp.stream_order(full.shape[0], x.device)]

    @staticmethod
    def backward(ctx, dy):
        cp = ctx.cp
        return dy[cp.local_index(ctx.total, dy.device)].contiguous(), None


# ------------------------------------------------------------------------------------------------ ring exchange
def _ring_exchange(send: torch.Tensor, cp: CP) -> tuple[torch.Tensor, list]:
    """Starts sending ``send`` to rank + 1 and receiving the same-shaped tensor from rank - 1; returns (buffer, requests)."""
    recv = torch.empty_like(send)
    nxt = dist.get_global_rank(cp.group, (cp.rank + 1) % cp.world) if cp.group is not None else (cp.rank + 1) % cp.world
    prv = dist.get_global_rank(cp.group, (cp.rank - 1) % cp.world) if cp.group is not None else (cp.rank - 1) % cp.world
    ops = [dist.P2POp(dist.isend, send, nxt, group=cp.group), dist.P2POp(dist.irecv, recv, prv, group=cp.group)]
    return recv, dist.batch_isend_irecv(ops)


def _wait(reqs) -> None:
    for r in reqs:
        r.wait()


def _row_meta(cu_seqlens: torch.Tensor, total: int, device) -> torch.Tensor:
    """Sequence id of every stream row (rows beyond the last boundary get an id of their own)."""
    rows = torch.arange(total, device=device)
    return torch.searchsorted(cu_seqlens[1:].to(device).long().contiguous(), rows, right=True)


def _block_scores(q, k, scale, q_rows, k_rows, q_seq, k_seq):
    """q [nq, hkv, rep, d], k [nk, hkv, d] -> masked scores [hkv, rep, nq, nk] in fp32 (-inf where invisible)."""
    s = torch.einsum("qhrd,khd->hrqk", q, k).float() * scale
    vis = (q_seq[:, None] == k_seq[None, :]) & (k_rows[None, :] <= q_rows[:, None])
    return s.masked_fill(~vis[None, None], float("-inf"))


class _RingAttention(torch.autograd.Function):
    Q_TILE = 1024

    @staticmethod
    def forward(ctx, q, k, v, rows, seq, cp: CP, scale: float):
        """q [n, hq, d]; k, v [n, hkv, d] of the local rows; ``rows`` [n] their stream positions; ``seq`` [n] their
        sequence ids. Returns the attention output [n, hq, d]."""
        n, hq, d = q.shape
        hkv = k.shape[1]
        rep = hq // hkv
        dev = q.device
        qg = q.reshape(n, hkv, rep, d)
        acc = torch.zeros((n, hkv, rep, d), dtype=torch.float32, device=dev)
        m = torch.full((n, hkv, rep), float("-inf"), dtype=torch.float32, device=dev)
        l = torch.zeros((n, hkv, rep), dtype=torch.float32, device=dev)
        # the travelling block: keys, values and the stream rows / sequence ids they belong to
        blk = torch.cat([k.reshape(n, -1), v.reshape(n, -1)], dim=1).contiguous()
        meta = torch.stack([rows, seq], dim=1).contiguous()
        for step in range(cp.world):
            if step + 1 < cp.world:
                nxt_blk, r1 = _ring_exchange(blk, cp)
                nxt_meta, r2 = _ring_exchange(meta, cp)
            kb = blk[:, : hkv * d].reshape(n, hkv, d)
            vb = blk[:, hkv * d :].reshape(n, hkv, d)
            k_rows, k_seq = meta[:, 0], meta[:, 1]
            if bool((k_rows.min() <= rows.max())):   # otherwise the whole block lies in the future of every local query
                for t0 in range(0, n, _RingAttention.Q_TILE):
                    t1 = min(n, t0 + _RingAttention.Q_TILE)
                    if bool(k_rows.min() > rows[t0:t1].max()):
                        continue
                    s = _block_scores(qg[t0:t1], kb, scale, rows[t0:t1], k_rows, seq[t0:t1], k_seq)      # [hkv, rep, tq, nk]
                    bm = s.amax(-1).permute(2, 0, 1)                                                      # [tq, hkv, rep]
                    new_m = torch.maximum(m[t0:t1], bm)
                    safe = torch.where(torch.isinf(new_m), torch.zeros_like(new_m), new_m)
                    p = torch.exp(s - safe.permute(1, 2, 0)[..., None])
                    alpha = torch.exp(m[t0:t1] - safe)
                    alpha = torch.where(torch.isinf(m[t0:t1]), torch.zeros_like(alpha), alpha)
                    l[t0:t1] = l[t0:t1] * alpha + p.sum(-1).permute(2, 0, 1)
                    acc[t0:t1] = acc[t0:t1] * alpha[..., None] + torch.einsum("hrqk,khd->qhrd", p.to(vb.dtype), vb).float()
                    m[t0:t1] = new_m
            if step + 1 < cp.world:
                _wait(r1)
                _wait(r2)
                blk, meta = nxt_blk, nxt_meta
        l_safe = torch.where(l == 0, torch.ones_like(l), l)
        out = (acc / l_safe[..., None]).to(q.dtype)
        lse = torch.where(l == 0, torch.full_like(m, float("-inf")), m + torch.log(l_safe))
        ctx.save_for_backward(q, k, v, out, lse, rows, seq)
        ctx.cp, ctx.scale = cp, scale
        return out.reshape(n, hq, d)

    @staticmethod
    def backward(ctx, d_out):
        q, k, v, out, lse, rows, seq = ctx.saved_tensors
        cp, scale = ctx.cp, ctx.scale
        n, hq, d = q.shape
        hkv = k.shape[1]
        rep = hq // hkv
        qg = q.reshape(n, hkv, rep, d)
        dog = d_out.reshape(n, hkv, rep, d)
        delta = (dog.float() * out.float()).sum(-1)                      # [n, hkv, rep]
        dq = torch.zeros((n, hkv, rep, d), dtype=torch.float32, device=q.device)
        # the block travels with its gradient accumulator: [k | v | dk | dv], the last two in fp32 precision
        blk = torch.cat([k.reshape(n, -1).float(), v.reshape(n, -1).float(), torch.zeros((n, 2 * hkv * d), device=q.device)], dim=1).contiguous()
        meta = torch.stack([rows, seq], dim=1).contiguous()
        W = hkv * d
        for step in range(cp.world):
            kb = blk[:, :W].reshape(n, hkv, d).to(q.dtype)
            vb = blk[:, W : 2 * W].reshape(n, hkv, d).to(q.dtype)
            dkb = blk[:, 2 * W : 3 * W].reshape(n, hkv, d)
            dvb = blk[:, 3 * W :].reshape(n, hkv, d)
            k_rows, k_seq = meta[:, 0], meta[:, 1]
            if bool((k_rows.min() <= rows.max())):
                for t0 in range(0, n, _RingAttention.Q_TILE):
                    t1 = min(n, t0 + _RingAttention.Q_TILE)
                    if bool(k_rows.min() > rows[t0:t1].max()):
                        continue
                    s = _block_scores(qg[t0:t1], kb, scale, rows[t0:t1], k_rows, seq[t0:t1], k_seq)
                    ls = lse[t0:t1].permute(1, 2, 0)[..., None]
                    p = torch.exp(s - torch.where(torch.isinf(ls), torch.zeros_like(ls), ls))
                    p = torch.where(torch.isinf(s), torch.zeros_like(p), p)                          # [hkv, rep, tq, nk]
                    dvb += torch.einsum("hrqk,qhrd->khd", p, dog[t0:t1].float())
                    dp = torch.einsum("qhrd,khd->hrqk", dog[t0:t1].float(), vb.float())
                    ds = p * (dp - delta[t0:t1].permute(1, 2, 0)[..., None]) * scale
                    dq[t0:t1] += torch.einsum("hrqk,khd->qhrd", ds, kb.float())
                    dkb += torch.einsum("hrqk,qhrd->khd", ds, qg[t0:t1].float())
            # pass the block (with its gradients) on; after cp hops it is back at its owner
            if cp.world > 1:
                nxt_blk, r1 = _ring_exchange(blk, cp)
                nxt_meta, r2 = _ring_exchange(meta, cp)
                _wait(r1)
                _wait(r2)
                blk, meta = nxt_blk, nxt_meta
        dk = blk[:, 2 * W : 3 * W].reshape(n, hkv, d).to(k.dtype)
        dv = blk[:, 3 * W :].reshape(n, hkv, d).to(v.dtype)
        return dq.reshape(n, hq, d).to(q.dtype), dk, dv, None, None, None, None


def cp_attention_varlen(qkv_local: torch.Tensor, cu_seqlens: torch.Tensor, cp: CP, hq: int, hkv: int, d: int,
                        scale: Optional[float] = None, total_rows: Optional[int] = None) -> torch.Tensor:
    """``qkv_local`` [T / cp, (hq + 2 hkv) d]: fused q, k, v of this rank's rows in local (zig-zag) order, already rotated.
    Returns the causal attention output of those rows [T / cp, hq d], computed with the ring."""
    n = qkv_local.shape[0]
    T = total_rows if total_rows is not None else n * cp.world
    dev = qkv_local.device
    rows = cp.local_index(T, dev)
    seq = _row_meta(cu_seqlens, T, dev)[rows]
    q = qkv_local[:, : hq * d].reshape(n, hq, d)
    k = qkv_local[:, hq * d : (hq + hkv) * d].reshape(n, hkv, d)
    v = qkv_local[:, (hq + hkv) * d :].reshape(n, hkv, d)
    scale = scale if scale is not None else d ** -0.5
    out = _RingAttention.apply(q.contiguous(), k.contiguous(), v.contiguous(), rows, seq, cp, float(scale))
    return out.reshape(n, hq * d)
