"""Operators used by the generation engine: paged KV cache write, paged decode attention, sampling."""

from __future__ import annotations

import math
import os
from typing import Optional

import torch

from . import lib as _L
from .lib import call, ptr, stream_ptr, use_native


def kv_cache_write(qkv: torch.Tensor, slots: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                   Hq: int, Hkv: int, D: int) -> None:
    """Scatters the k and v heads of a fused [T, (Hq+2Hkv)*D] projection into the paged cache.

    ``slots`` [T] int64: block * block_size + offset of each token (negative: skip).
    Cache tensors are [num_blocks, Hkv, block_size, D].
    """
    block_size = k_cache.shape[2]
    if not use_native(qkv):
        T = qkv.shape[0]
        k = qkv[:, Hq * D : (Hq + Hkv) * D].reshape(T, Hkv, D)
        v = qkv[:, (Hq + Hkv) * D :].reshape(T, Hkv, D)
        ok = slots >= 0
        blk = (slots[ok] // block_size).long()
        off = (slots[ok] % block_size).long()
        k_cache[blk, :, off] = k[ok]
        v_cache[blk, :, off] = v[ok]
        return
    call("rlb_kv_cache_write", ptr(qkv), ptr(slots), ptr(k_cache), ptr(v_cache), qkv.shape[0], Hq, Hkv, D,
         block_size, qkv.stride(0), k_cache.shape[0], ptr(_L.status_word(qkv.device)), stream_ptr())


def rope_kv_cache_write(qkv: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, slots: torch.Tensor, k_cache: torch.Tensor,
                        v_cache: torch.Tensor, Hq: int, Hkv: int, D: int) -> torch.Tensor:
    """Rotary embedding of q and k (in place on CUDA) and the cache scatter of k and v in one launch; returns the rotated
    fused rows."""
    if not use_native(qkv):
        from rl_b200.ops import functional as F

        qkv = F.rope(qkv, positions, inv_freq, Hq + Hkv, D)
        kv_cache_write(qkv, slots, k_cache, v_cache, Hq, Hkv, D)
        return qkv
    call("rlb_rope_kv_cache_write", ptr(qkv), ptr(positions.to(torch.int32)), ptr(inv_freq), ptr(slots), ptr(k_cache), ptr(v_cache),
         qkv.shape[0], Hq, Hkv, D, k_cache.shape[2], qkv.stride(0), k_cache.shape[0], ptr(_L.status_word(qkv.device)), stream_ptr())
    return qkv


def decode_scratch_sizes(B: int, Hq: int, num_splits: int, D: int = 128) -> tuple[int, int]:
    return B * Hq * num_splits * D, B * Hq * num_splits * 2


def skinny_static_weights(on: bool) -> int:
    """Tells the decode GEMM whether its weight operand is never written by the kernel launched just before it (true during a
    generation phase); returns the previous setting."""
    from .lib import lib

    return int(lib().rlb_gemm_skinny_static_weights(1 if on else 0))


def choose_splits(B: int, Hkv: int, max_len: int, block_size: int, sm_count: int = 148) -> int:
    """Enough KV splits to put ~2 CTAs on every SM, never finer than one cache block per split."""
    forced = os.environ.get("RLB_DECODE_SPLITS")
    if forced:
        return max(1, int(forced))
    ctas = max(1, B * Hkv)
    want = max(1, (2 * sm_count + ctas - 1) // ctas)
    return int(max(1, min(want, max(1, max_len // max(block_size, 128)), 32)))


def _paged_decode_gather(q, k_cache, v_cache, block_table, seq_lens, Hq, Hkv, D, scale, out, rows_per_chunk: int = 64, window: int = 0):
    """Decode attention for head dimensions the native kernels do not cover (they are built for 128): the paged keys and
    values of a chunk of sequences are gathered through the block table and attended with batched matmuls. No host
    synchronisation and static shapes, so it can be captured in a CUDA graph like the native path."""
    B, nb = q.shape[0], block_table.shape[1]
    bs, g = k_cache.shape[2], Hq // Hkv
    T = nb * bs
    ar = torch.arange(T, device=q.device)
    for r0 in range(0, B, rows_per_chunk):
        r1 = min(B, r0 + rows_per_chunk)
        bt = block_table[r0:r1].long()
        k = k_cache[bt].permute(0, 2, 1, 3, 4).reshape(r1 - r0, Hkv, T, D)
        v = v_cache[bt].permute(0, 2, 1, 3, 4).reshape(r1 - r0, Hkv, T, D)
        qb = (q[r0:r1, : Hq * D].reshape(r1 - r0, Hkv, g, D).float() * scale).to(k.dtype)
        s_ = torch.matmul(qb, k.transpose(2, 3)).float()
        live = ar[None, :] < seq_lens[r0:r1, None]
        if window:
            live = live & (ar[None, :] >= seq_lens[r0:r1, None] - window)
        s_ = s_.masked_fill(~live[:, None, None, :], float("-inf"))
        p = torch.nan_to_num(torch.softmax(s_, dim=-1), nan=0.0)   # rows without context (padding rows) give zeros
        out[r0:r1] = torch.matmul(p.to(v.dtype), v).reshape(r1 - r0, Hq * D).to(out.dtype)
    return out


def paged_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                 seq_lens: torch.Tensor, Hq: int, Hkv: int, D: int, *, scale: Optional[float] = None,
                 num_splits: int = 1, scratch: Optional[tuple[torch.Tensor, torch.Tensor]] = None,
                 out: Optional[torch.Tensor] = None, window: int = 0) -> torch.Tensor:
    """Attention of one query token per sequence against its paged KV. ``q`` [B, Hq*D] (rows may be strided). ``window`` > 0:
    only the last ``window`` cached tokens are visible (sliding-window layers; served by the gather path)."""
    B = q.shape[0]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    block_size = k_cache.shape[2]
    if out is None:
        out = torch.empty((B, Hq * D), dtype=q.dtype, device=q.device)
    if not use_native(q):
        g = Hq // Hkv
        for b in range(B):
            n = int(seq_lens[b])
            if n == 0:
                out[b] = 0
                continue
            nb = (n + block_size - 1) // block_size
            blocks = block_table[b, :nb].long()
            lo = max(0, n - window) if window else 0
            k = k_cache[blocks].permute(1, 0, 2, 3).reshape(Hkv, nb * block_size, D)[:, lo:n].float()
            v = v_cache[blocks].permute(1, 0, 2, 3).reshape(Hkv, nb * block_size, D)[:, lo:n].float()
            qb = q[b, : Hq * D].reshape(Hkv, g, D).float() * scale
            p = torch.softmax(qb @ k.transpose(1, 2), dim=-1)
            out[b] = (p @ v).reshape(Hq * D).to(out.dtype)
        return out
    if D != 128 or window:
        return _paged_decode_gather(q, k_cache, v_cache, block_table, seq_lens, Hq, Hkv, D, scale, out, window=window)
    po = pml = None
    if num_splits > 1:
        if scratch is None:
            no, nml = decode_scratch_sizes(B, Hq, num_splits, D)
            scratch = (torch.empty(no, dtype=torch.float32, device=q.device),
                       torch.empty(nml, dtype=torch.float32, device=q.device))
        po, pml = scratch
    kernel = os.environ.get("RLB_DECODE_KERNEL", "mma")
    if kernel == "mma" and D == 128 and Hq // Hkv <= 8 and (block_size in (16, 32, 64) or block_size % 128 == 0):
        # tensor-core flash-decoding kernel (tcgen05: QK^T and PV as MMAs over 128-token tiles)
        call("rlb_paged_decode_mma", ptr(q), q.stride(0), ptr(k_cache), ptr(v_cache), k_cache.shape[0], ptr(block_table),
             block_table.stride(0), ptr(seq_lens), B, Hq, Hkv, D, block_size, scale, num_splits, ptr(po), ptr(pml), ptr(out),
             out.stride(0), ptr(_L.status_word(q.device)), stream_ptr())
        return out
    if block_size in (16, 32) or block_size % 64 == 0:
        # CUDA-core TMA-pipelined kernel (the plain-load kernel below remains for other block sizes)
        call("rlb_paged_decode_tma", ptr(q), q.stride(0), ptr(k_cache), ptr(v_cache), k_cache.shape[0], ptr(block_table),
             block_table.stride(0), ptr(seq_lens), B, Hq, Hkv, D, block_size, scale, num_splits, ptr(po), ptr(pml), ptr(out),
             out.stride(0), ptr(_L.status_word(q.device)), stream_ptr())
        return out
    call("rlb_paged_decode", ptr(q), q.stride(0), ptr(k_cache), ptr(v_cache), ptr(block_table), block_table.stride(0),
         ptr(seq_lens), B, Hq, Hkv, D, block_size, scale, num_splits, ptr(po), ptr(pml), ptr(out), out.stride(0),
         stream_ptr())
    return out


def sample(logits: torch.Tensor, *, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0, greedy: bool = False,
           seed: int = 0, step: int = 0, temps: Optional[torch.Tensor] = None, top_ks: Optional[torch.Tensor] = None,
           top_ps: Optional[torch.Tensor] = None, generator: Optional[torch.Generator] = None,
           step_tensor: Optional[torch.Tensor] = None, out: Optional[tuple[torch.Tensor, torch.Tensor]] = None,
           row_keys: Optional[torch.Tensor] = None):
    """Draws one token per row of ``logits`` [B, V] and returns (tokens int32 [B], logprobs fp32 [B]); the
    log-probabilities are those of the distribution after temperature / top-k / top-p."""
    B, V = logits.shape
    if not use_native(logits):
        z = logits.float()
        t = temperature if temperature > 0 else 1.0
        z = z / t
        if top_k and 0 < top_k < V:
            kth = torch.topk(z, top_k, dim=-1).values[:, -1:]
            z = z.masked_fill(z < kth, float("-inf"))
        if top_p < 1.0:
            sz, si = torch.sort(z, dim=-1, descending=True)
            probs = torch.softmax(sz, dim=-1)
            cum = probs.cumsum(-1)
            drop = (cum - probs) >= top_p  # keep the smallest prefix whose mass reaches top_p
            sz = sz.masked_fill(drop, float("-inf"))
            z = torch.full_like(z, float("-inf")).scatter(-1, si, sz)
        logp = torch.log_softmax(z, dim=-1)
        if greedy or temperature <= 0:
            tok = logp.argmax(-1)
        elif row_keys is not None:
            # one generator per row, seeded by (seed, key): the draw does not depend on the batch composition
            tok = torch.empty(B, dtype=torch.long)
            for i, k in enumerate(row_keys.tolist()):
                g = torch.Generator().manual_seed((seed * 0x9E3779B97F4A7C15 + k * 0xBF58476D1CE4E5B9) % (2**63))
                tok[i] = torch.multinomial(logp[i].exp(), 1, generator=g)
        else:
            tok = torch.multinomial(logp.exp(), 1, generator=generator).squeeze(-1)
        return tok.to(torch.int32), logp.gather(-1, tok.long().unsqueeze(-1)).squeeze(-1)
    assert logits.stride(1) == 1
    if out is None:
        tok = torch.empty(B, dtype=torch.int32, device=logits.device)
        lp = torch.empty(B, dtype=torch.float32, device=logits.device)
    else:
        tok, lp = out
    dtype = 0 if logits.dtype == torch.float32 else 1
    assert logits.dtype in (torch.float32, torch.bfloat16)
    # step_tensor: a 1-element int64 CUDA tensor holding the draw counter, for launches replayed from a CUDA graph
    call("rlb_sample", ptr(logits), dtype, logits.stride(0), B, V, ptr(temps), ptr(top_ks), ptr(top_ps),
         float(temperature), int(top_k), float(top_p), int(greedy), seed & (2**64 - 1), step & (2**64 - 1),
         ptr(step_tensor), ptr(row_keys), ptr(tok), ptr(lp), stream_ptr())
    return tok, lp


def skinny_linear(x: torch.Tensor, w: torch.Tensor, *, out: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16,
                  bias: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
                  ssq_in: Optional[torch.Tensor] = None, eps: float = 1e-6, ssq_out: Optional[torch.Tensor] = None,
                  norm_w: Optional[torch.Tensor] = None, out2: Optional[torch.Tensor] = None, swiglu: bool = False) -> torch.Tensor:
    """Decode-sized projection (at most 256 rows) with the epilogue fusions of ``rlb_gemm_skinny_fused``.

    ``ssq_in`` [tiles, stride]: ``x`` is ``h * w_norm`` and the output rows are scaled by the reciprocal RMS of ``h`` built
    from these partial sums (RMSNorm folded into the projection). ``ssq_out`` + ``norm_w`` + ``out2``: also writes
    ``out2 = y * norm_w`` and the partial sums of squares of ``y`` for the next norm. ``swiglu``: ``w`` is [gate | up] and the
    result is ``silu(x gate^T) * (x up^T)``. CPU tensors run the fp32 statement of the same math."""
    M, K = x.shape
    N = w.shape[0] // 2 if swiglu else w.shape[0]
    if not use_native(x):
        xf = x.float()
        y = xf @ w.float().t()
        if ssq_in is not None:
            y = y * torch.rsqrt(ssq_in[:, :M].sum(0) / K + eps)[:, None]
        if swiglu:
            y = torch.nn.functional.silu(y[:, :N]) * y[:, N:]
        if bias is not None:
            y = y + bias.float()
        if residual is not None:
            y = y + residual.float()
        y = y.to(out_dtype)
        if ssq_out is not None:
            yf = y.float()
            out2.copy_((yf * norm_w.float()).to(out2.dtype))
            tiles = (N + 127) // 128
            pad = torch.zeros((M, tiles * 128), dtype=torch.float32)
            pad[:, :N] = yf * yf
            ssq_out[:tiles, :M] = pad.view(M, tiles, 128).sum(-1).t()
        if out is not None:
            out.copy_(y)
            return out
        return y
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    if bias is not None and bias.dtype != torch.float32:
        bias = bias.float()
    call("rlb_gemm_skinny_fused", ptr(x), ptr(w), ptr(out), M, N, K, x.stride(0), w.stride(0), out.stride(0),
         int(out.dtype == torch.float32), ptr(bias), ptr(residual), residual.stride(0) if residual is not None else 0, 0,
         ptr(ssq_in), ssq_in.shape[0] if ssq_in is not None else 0, ssq_in.stride(0) if ssq_in is not None else 0, float(eps),
         ptr(ssq_out), ssq_out.stride(0) if ssq_out is not None else 0, ptr(norm_w), ptr(out2),
         out2.stride(0) if out2 is not None else 0, int(swiglu), ptr(_L.status_word(x.device)), stream_ptr())
    return out


def decode_advance(st: dict, B: int, block_size: int, max_window: int, n_stop: int) -> None:
    """Advances the device-resident decode-step inputs of ``B`` rows after sampling (``rlb_decode_advance``): ``st`` is the
    engine's dict of fixed-address step tensors."""
    bt = st["block_table"]
    call("rlb_decode_advance", ptr(st["tok"]), ptr(st["lp"]), ptr(st["ids"]), ptr(st["positions"]), ptr(st["seq_lens"]),
         ptr(st["slots"]), ptr(st["keys"]), ptr(bt), bt.stride(0), ptr(st["active"]), ptr(st["remaining"]), ptr(st["produced"]),
         ptr(st["stop_ids"]), int(n_stop), ptr(st["out_tok"]), ptr(st["out_lp"]), st["out_tok"].stride(0), int(max_window),
         ptr(st["win_step"]), B, int(block_size), stream_ptr())


def block_copy(k_cache: torch.Tensor, v_cache: torch.Tensor, src: torch.Tensor, dst: torch.Tensor) -> None:
    """Copies whole cache blocks ``src[i] -> dst[i]`` in both caches (copy-on-write of a shared prompt's tail block)."""
    n = src.numel()
    if n == 0:
        return
    if not use_native(k_cache):
        k_cache[dst.long()] = k_cache[src.long()]
        v_cache[dst.long()] = v_cache[src.long()]
        return
    elems = k_cache[0].numel()
    call("rlb_block_copy", ptr(k_cache), ptr(v_cache), ptr(src), ptr(dst), n, elems, stream_ptr())


def gather_rows(x: torch.Tensor, idx: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[i] = x[idx[i]] for a bf16 [T, d] matrix (last-token hidden states of a packed batch)."""
    if not use_native(x):
        return x[idx.long()]
    n, d = idx.numel(), x.shape[1]
    if out is None:
        out = torch.empty((n, d), dtype=x.dtype, device=x.device)
    call("rlb_gather_rows", ptr(x), ptr(idx), ptr(out), n, d, x.stride(0), out.stride(0), stream_ptr())
    return out
