"""Vocabulary-parallel log-probabilities: every tensor-parallel rank owns a contiguous slice of the vocabulary rows
of the output projection, computes softmax statistics over its slice with the fused projection kernel (the
``[T, V/tp]`` logits are never stored), and the ranks exchange three floats per token (log-sum-exp, E[z], target logit).

Backward recomputes the local logits slice chunk by chunk into dZ, accumulates dW of the slice and produces the partial
dH that is reduce-scattered (sequence parallel) or all-reduced over the group. This is the role of
``DistributedLogprob`` / ``ChunkedDistributedHiddenStatesToLogprobs`` in the reference
(nemo_rl/distributed/model_utils.py:1035-1280, :2137-2316).
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from rl_b200.ops import functional as F
from rl_b200.ops import lib as _L
from rl_b200.ops.lib import call, ptr, stream_ptr, use_native
from rl_b200.parallel.tensor import TP, all_gather_rows, all_reduce_, reduce_scatter_rows

BF16 = torch.bfloat16
CHUNK = 8192


def _local_stats(h, w, tg_local, inv_temp):
    """Per-row (lse, entropy, target logit or 0) of softmax over this rank's vocabulary slice."""
    M, K = h.shape
    N = w.shape[0]
    dev = h.device
    if use_native(h):
        parts = _L.lib().rlb_gemm_num_n_tiles(N)
        pm = torch.empty((3, parts, M), dtype=torch.float32, device=dev)
        tl = torch.zeros(M, dtype=torch.float32, device=dev)
        out = torch.empty((3, M), dtype=torch.float32, device=dev)
        call("rlb_lm_head_logprob", ptr(h), ptr(w), M, N, K, h.stride(0), w.stride(0), ptr(tg_local), inv_temp,
             ptr(pm[0]), ptr(pm[1]), ptr(pm[2]), ptr(tl), ptr(out[2]), ptr(out[1]), ptr(out[0]), ptr(_L.status_word(dev)), stream_ptr())
        out[2].copy_(tl)
        return out
    z = (h.float() @ w.float().t()) * inv_temp
    lse = torch.logsumexp(z, dim=-1)
    ent = lse - (torch.softmax(z, dim=-1) * z).sum(-1)
    inside = (tg_local >= 0) & (tg_local < N)
    tl = torch.where(inside, z.gather(-1, tg_local.clamp(0, N - 1).long().unsqueeze(-1)).squeeze(-1), torch.zeros_like(lse))
    return torch.stack([lse, ent, tl])


class _VocabParallelLogprob(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h_in, w, targets, vocab_start, inv_temp, want_entropy, tp: TP):
        sp = tp.sequence_parallel
        h = all_gather_rows(h_in, tp.group, tp.world) if sp else h_in
        h = h if h.stride(-1) == 1 else h.contiguous()
        N = w.shape[0]
        tg = (targets.to(torch.int64) - vocab_start)
        tg = torch.where((tg >= 0) & (tg < N), tg, torch.full_like(tg, -1)).to(torch.int32).contiguous()
        st = _local_stats(h, w, tg, inv_temp)                      # [3, M]
        allst = all_gather_rows(st.unsqueeze(0), tp.group, tp.world)  # [tp, 3, M]
        lse_r, ent_r, tl_r = allst[:, 0], allst[:, 1], allst[:, 2]
        lse = torch.logsumexp(lse_r, dim=0)
        wgt = torch.exp(lse_r - lse)                                # share of the probability mass per rank
        ez = (wgt * (lse_r - ent_r)).sum(0)                         # E[z] over the whole vocabulary
        ent = lse - ez
        logp = tl_r.sum(0) - lse
        ctx.save_for_backward(h_in if sp else h, w, tg, lse, ent)
        ctx.tp, ctx.inv_temp, ctx.want_entropy = tp, inv_temp, want_entropy
        return logp, (ent if want_entropy else None)

    @staticmethod
    def backward(ctx, dlogp, dent):
        h_saved, w, tg, lse, ent = ctx.saved_tensors
        tp = ctx.tp
        sp = tp.sequence_parallel
        h = all_gather_rows(h_saved, tp.group, tp.world) if sp else h_saved
        M, K = h.shape
        N = w.shape[0]
        dev = h.device
        coef = dlogp.float().contiguous()
        ecoef = dent.float().contiguous() if (dent is not None and ctx.want_entropy) else None
        main_grad = getattr(w, "main_grad", None)
        need_w = ctx.needs_input_grad[1]
        dh = torch.empty((M, K), dtype=h.dtype, device=dev)
        dw = None
        if use_native(h):
            if need_w and main_grad is None:
                dw = torch.zeros((N, K), dtype=torch.float32, device=dev)
            target = main_grad if main_grad is not None else dw
            dz = torch.empty((min(CHUNK, M), N), dtype=BF16, device=dev)
            for s in range(0, M, CHUNK):
                e = min(M, s + CHUNK)
                dzc = dz[: e - s]
                call("rlb_lm_head_dlogits", ptr(h[s:e]), ptr(w), ptr(dzc), e - s, N, K, h.stride(0), w.stride(0), dzc.stride(0),
                     ptr(tg[s:e]), ctx.inv_temp, ptr(lse[s:e]), ptr(coef[s:e]), ptr(ecoef[s:e]) if ecoef is not None else None,
                     ptr(ent[s:e]), ptr(_L.status_word(dev)), stream_ptr())
                F.gemm(dzc, w, b_mn=True, out=dh[s:e])
                if target is not None:
                    F.gemm(dzc, h[s:e], a_mn=True, b_mn=True, out=target, accumulate=True)
            if dw is not None:
                dw = dw.to(w.dtype)
        else:
            z = (h.float() @ w.float().t()) * ctx.inv_temp
            p = torch.exp(z - lse.unsqueeze(-1))
            onehot = torch.zeros_like(p)
            inside = tg >= 0
            onehot[inside, tg[inside].long()] = 1.0
            dz = coef.unsqueeze(-1) * (onehot - p)
            if ecoef is not None:  # dH/dz_j = -p_j (z_j - E[z]) with E[z] = lse - H
                dz = dz - ecoef.unsqueeze(-1) * p * (z - (lse - ent).unsqueeze(-1))
            dz = dz * ctx.inv_temp
            dh = (dz @ w.float()).to(h.dtype)
            if need_w:
                g = dz.t() @ h.float()
                if main_grad is not None:
                    main_grad.add_(g.to(main_grad.dtype))
                else:
                    dw = g.to(w.dtype)
        dh = reduce_scatter_rows(dh, tp.group, tp.world, tp.rank) if sp else all_reduce_(dh, tp.group, tp.world)
        return dh, dw, None, None, None, None, None


def vocab_parallel_logprobs(h: torch.Tensor, w_shard: torch.Tensor, targets: torch.Tensor, tp: TP, vocab_start: int,
                            temperature: float = 1.0, want_entropy: bool = False):
    """``h``: this rank's row shard (sequence parallel) or all rows (replicated); ``w_shard`` [V/tp, d] rows
    ``[vocab_start, vocab_start + V/tp)``; ``targets``: global token ids for ALL rows. Returns (logp [T], entropy | None)."""
    if tp.world == 1:
        return F.lm_head_logprobs(h, w_shard, targets, temperature, want_entropy)
    return _VocabParallelLogprob.apply(h, w_shard, targets, int(vocab_start), 1.0 / temperature, want_entropy, tp)


# --------------------------------------------------------------------------------------------- vocab-parallel argmax / top-k
def vocab_parallel_topk(logits_shard: torch.Tensor, k: int, tp: TP, vocab_start: int):
    """Top-k over a vocabulary that is sharded across the tensor-parallel group: every rank takes the top-k of its slice,
    the candidates ([T, k] values + global ids per rank) are all-gathered and reduced to the global top-k
    (nemo_rl/distributed/model_utils.py ``distributed_vocab_topk``). Returns (values [T, k], global ids [T, k])."""
    kk = min(k, logits_shard.shape[-1])
    v, i = torch.topk(logits_shard.float(), kk, dim=-1)
    i = i + vocab_start
    if tp.world == 1:
        return v, i
    allv = all_gather_rows(v.t().contiguous(), tp.group, tp.world).t()   # [T, tp * kk]
    alli = all_gather_rows(i.t().contiguous(), tp.group, tp.world).t()
    tv, pos = torch.topk(allv, min(k, allv.shape[-1]), dim=-1)
    return tv, alli.gather(-1, pos)


def vocab_parallel_argmax(logits_shard: torch.Tensor, tp: TP, vocab_start: int) -> torch.Tensor:
    """Global argmax token id per row (greedy decoding over a sharded vocabulary)."""
    return vocab_parallel_topk(logits_shard, 1, tp, vocab_start)[1][:, 0]


# ------------------------------------------------------------------------- log-probabilities under top-k / top-p
class _VocabToRows(torch.autograd.Function):
    """Vocabulary-parallel logits [R, V / tp] (all rows, this rank's columns) -> row-parallel logits [R / tp, V] (this
    rank's rows, all columns) with one all-to-all; the backward pass is the reverse exchange
    (the vocab <-> sequence all-to-all of nemo_rl/distributed/model_utils.py:2465-2565)."""

    @staticmethod
    def forward(ctx, z, tp: TP):
        R, n = z.shape
        W = tp.world
        assert R % W == 0
        ctx.tp, ctx.shape = tp, (R, n)
        send = z.reshape(W, R // W, n).contiguous()                  # chunk j: the rows rank j will own
        recv = torch.empty_like(send)                                # chunk i: my rows, rank i's columns
        dist.all_to_all_single(recv.view(-1), send.view(-1), group=tp.group)
        return recv.permute(1, 0, 2).reshape(R // W, W * n)

    @staticmethod
    def backward(ctx, dy):
        tp = ctx.tp
        R, n = ctx.shape
        W = tp.world
        send = dy.reshape(R // W, W, n).permute(1, 0, 2).contiguous()
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv.view(-1), send.view(-1), group=tp.group)
        return recv.reshape(R, n), None


def vocab_parallel_filtered_logprobs(h: torch.Tensor, w_shard: torch.Tensor, targets: torch.Tensor, tp: TP, temperature: float,
                                     top_k, top_p, chunk_rows: int = 2048) -> torch.Tensor:
    """log p(target) under the sampler's processed distribution (temperature, top-k, then top-p) with a vocabulary-parallel
    output projection, without any rank ever holding ``[T, V]``: ``chunk_rows`` rows at a time, each rank projects the
    chunk onto its vocabulary slice, an all-to-all turns the column shards into row shards with the full vocabulary,
    every rank filters and scores its rows, and the per-row results are gathered. ``h``: all rows (or this rank's rows
    when ``tp.sequence_parallel``); ``targets`` [T]. Returns [T] fp32, -1e4 where the target is outside the kept set.
    (DistributedLogprobWithSampling, nemo_rl/distributed/model_utils.py:383-510.)"""
    from rl_b200.algorithms.sampling_utils import apply_top_k_top_p
    from rl_b200.parallel.tensor import column_linear, gather_rows

    W = tp.world
    T = targets.shape[0]
    rows_tp = TP(tp.group, tp.rank, W)
    inv_t = temperature if temperature > 0 else 1.0

    def score(z, tg):
        z, _ = apply_top_k_top_p(z / inv_t, top_k, top_p)
        lp = torch.log_softmax(z, dim=-1).gather(-1, tg.long()[:, None])[:, 0]
        return torch.where(torch.isfinite(lp), lp, torch.full_like(lp, -1e4))

    out = []
    if tp.sequence_parallel:
        # h holds this rank's rows: the gathering projection returns the chunk's rows rank-major, so the all-to-all hands
        # every rank exactly its own rows back, now with the whole vocabulary
        per = h.shape[0]
        mine = targets[tp.rank * per : (tp.rank + 1) * per]
        step = max(1, chunk_rows // W)
        for r0 in range(0, per, step):
            z = _VocabToRows.apply(column_linear(h[r0 : r0 + step], w_shard, None, tp).float(), tp)
            out.append(score(z, mine[r0 : r0 + step]))
        return gather_rows(torch.cat(out), rows_tp)
    step = max(W, chunk_rows // W * W)
    for r0 in range(0, T, step):
        hc, tg = h[r0 : r0 + step], targets[r0 : r0 + step]
        n = hc.shape[0]
        pad = (-n) % W
        if pad:
            hc = torch.cat([hc, hc.new_zeros((pad, hc.shape[1]))])
            tg = torch.cat([tg, tg.new_zeros(pad)])
        z = _VocabToRows.apply(column_linear(hc, w_shard, None, tp).float(), tp)           # [rows / W, V]
        per = (n + pad) // W
        out.append(gather_rows(score(z, tg[tp.rank * per : (tp.rank + 1) * per]), rows_tp)[:n])
    return torch.cat(out)
