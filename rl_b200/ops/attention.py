"""Native varlen causal attention (tcgen05 flash attention) with autograd.

Importing this module installs the native implementation behind :func:`rl_b200.ops.functional.attention_varlen` for
CUDA tensors with head dimension 128 or 64 (one instantiation of the kernels each; the head-dimension-64 entry points carry
the suffix ``_d64``). Other head dimensions use the PyTorch restatement.
"""

from __future__ import annotations

import torch

from . import functional as F
from . import lib as _L
from .lib import C, call, ptr, stream_ptr

_L.register("rlb_flash_attn_fwd", [_L.P, _L.L, _L.P, _L.I, _L.I, _L.I, _L.I, _L.I, _L.F, _L.P, _L.L, _L.P, _L.I, _L.P, _L.P])
_L.register("rlb_attn_delta", [_L.P, _L.P, _L.P, _L.I, _L.I, _L.L, _L.L, _L.P])
_L.register("rlb_flash_attn_bwd", [_L.P, _L.L, _L.P, _L.L, _L.P, _L.P, _L.P, _L.I, _L.I, _L.I, _L.I, _L.I, _L.F, _L.P, _L.L,
                                   _L.I, _L.I, _L.P, _L.P])
for _n in ("rlb_flash_attn_fwd", "rlb_attn_delta", "rlb_flash_attn_bwd"):
    _L.register(_n + "_d64", _L._SIGS[_n])
NATIVE_HEAD_DIMS = (64, 128)


def _sfx(D: int) -> str:
    return "" if D == 128 else f"_d{D}"


def flash_fwd(qkv: torch.Tensor, cu_seqlens: torch.Tensor, Hq: int, Hkv: int, D: int, scale: float, want_lse: bool = True):
    T = qkv.shape[0]
    B = cu_seqlens.numel() - 1
    out = torch.empty((T, Hq * D), dtype=qkv.dtype, device=qkv.device)
    lse = torch.empty((Hq, T), dtype=torch.float32, device=qkv.device) if want_lse else None
    max_tiles = (T + 127) // 128 + B
    call("rlb_flash_attn_fwd" + _sfx(D), ptr(qkv), qkv.stride(0), ptr(cu_seqlens), B, T, Hq, Hkv, D, scale, ptr(out), out.stride(0),
         ptr(lse), max_tiles, ptr(_L.status_word(qkv.device)), stream_ptr())
    return out, lse


def _has_native_bwd() -> bool:
    return hasattr(_L.lib(), "rlb_flash_attn_bwd")


class _FlashAttn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, cu_seqlens, max_seqlen, Hq, Hkv, D, scale):
        out, lse = flash_fwd(qkv, cu_seqlens, Hq, Hkv, D, scale)
        ctx.save_for_backward(qkv, cu_seqlens, out, lse)
        ctx.meta = (max_seqlen, Hq, Hkv, D, scale)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, cu, out, lse = ctx.saved_tensors
        max_seqlen, Hq, Hkv, D, scale = ctx.meta
        dout = dout.contiguous()
        if _has_native_bwd():
            T = qkv.shape[0]
            B = cu.numel() - 1
            dqkv = torch.empty_like(qkv)
            delta = torch.empty((Hq, T), dtype=torch.float32, device=qkv.device)
            call("rlb_attn_delta" + _sfx(D), ptr(dout), ptr(out), ptr(delta), T, Hq, dout.stride(0), out.stride(0), stream_ptr())
            call("rlb_flash_attn_bwd" + _sfx(D), ptr(qkv), qkv.stride(0), ptr(dout), dout.stride(0), ptr(lse), ptr(delta), ptr(cu), B, T,
                 Hq, Hkv, D, scale, ptr(dqkv), dqkv.stride(0), (T + 127) // 128 + B, (T + 63) // 64 + B,
                 ptr(_L.status_word(qkv.device)), stream_ptr())
            return dqkv, None, None, None, None, None, None
        # interim: differentiate the PyTorch restatement
        with torch.enable_grad():
            x = qkv.detach().requires_grad_()
            y = F._attention_ref(x, cu, Hq, Hkv, D, scale)
            (g,) = torch.autograd.grad(y, x, dout)
        return g, None, None, None, None, None, None


def attention_native(qkv, cu_seqlens, max_seqlen, Hq, Hkv, D, scale):
    if D not in NATIVE_HEAD_DIMS or qkv.dtype != torch.bfloat16 or not hasattr(_L.lib(), "rlb_flash_attn_fwd" + _sfx(D)):
        return F._attention_ref(qkv, cu_seqlens, Hq, Hkv, D, scale)
    cu = cu_seqlens.to(torch.int32)
    if qkv.stride(-1) != 1:
        qkv = qkv.contiguous()
    if torch.is_grad_enabled() and qkv.requires_grad:
        return _FlashAttn.apply(qkv, cu, max_seqlen, Hq, Hkv, D, scale)
    return flash_fwd(qkv, cu, Hq, Hkv, D, scale, want_lse=False)[0]


def install() -> None:
    if _L.available() and hasattr(_L.lib(), "rlb_flash_attn_fwd"):
        F.set_attention_impl(attention_native)


install()
