"""Low-precision rollout: the engine serves quantised copies of the trainer's bf16 linear weights.

``mxfp8`` (1 x 32 blocks, E8M0 scales): weights are quantised after every refit, activations on the fly, and the product
runs on the block-scaled tensor-core GEMM (``csrc/gemm_mxfp8.cu``). ``fp8`` (128 x 128 blocks, fp32 de-scales): weights
only; they are expanded to bf16 for the GEMM (storage and refit traffic shrink, arithmetic stays bf16). The trainer keeps
training and scoring in bf16; the importance-sampling correction of the loss absorbs the gap between the two policies, as
in the reference's FP8 rollout (nemo_rl/models/generation/vllm/quantization/fp8.py:37-59, :533-620, :832-858).

The quantised copies live in buffers that are allocated once and refreshed in place, so captured decode graphs stay valid
across refits.
"""

from __future__ import annotations

from contextlib import contextmanager
from typing import Optional

import torch

from rl_b200.ops import quant as Q

LINEAR_LEAVES = ("qkv_proj", "o_proj", "gate_up_proj", "down_proj")
_ACTIVE = {"on": False}


def is_active() -> bool:
    return _ACTIVE["on"]


@contextmanager
def quantized_inference(on: bool = True):
    """Inside this block ``rl_b200.ops.functional.linear`` uses the quantised copy of a weight that has one."""
    prev = _ACTIVE["on"]
    _ACTIVE["on"] = bool(on)
    try:
        yield
    finally:
        _ACTIVE["on"] = prev


def _eligible(name: str, p: torch.Tensor, kind: str) -> bool:
    leaf = name.rsplit(".", 1)[-1]
    if p.dim() != 2 or leaf not in LINEAR_LEAVES:
        return False
    return p.shape[1] % 128 == 0 and p.shape[0] % 8 == 0


@torch.no_grad()
def quantize_model(model, kind: str) -> dict:
    """(Re)fills the quantised copies of every eligible linear weight of ``model``; returns byte counts."""
    assert kind in ("mxfp8", "fp8")
    n = raw = packed = 0
    for name, p in model.named_parameters():
        if not _eligible(name, p, kind):
            continue
        w = p.detach()
        if w.dtype != torch.bfloat16:
            w = w.to(torch.bfloat16)
        if kind == "mxfp8":
            q, s = Q.quantize_mxfp8(w) if w.is_cuda else Q.quantize_mxfp8_ref(w)
            s = Q.swizzle_mx_scales(s) if w.is_cuda else s
        else:
            q, s = Q.quantize_fp8_blockwise(w) if w.is_cuda else Q.quantize_fp8_blockwise_ref(w)
        cur = getattr(p, "_rlb_q", None)
        if cur is not None and cur[0] == kind and cur[1].shape == q.shape and cur[2].shape == s.shape:
            cur[1].copy_(q)
            cur[2].copy_(s)
        else:
            p._rlb_q = (kind, q, s)
        if kind == "fp8" and w.is_cuda:
            # No block-128 FP8 GEMM exists here: the rollout computes with the fp8-rounded weights expanded to bf16 once per
            # refit (same numbers as expanding on every call, at the bf16 kernels' speed; costs a bf16 copy per weight).
            wd = Q.dequantize_fp8_blockwise(p._rlb_q[1], p._rlb_q[2])
            old = getattr(p, "_rlb_q_bf16", None)
            if old is not None and old.shape == wd.shape:
                old.copy_(wd)
            else:
                p._rlb_q_bf16 = wd
        n += 1
        raw += w.numel() * 2
        packed += q.numel() * q.element_size() + s.numel() * s.element_size()
    return dict(tensors=n, bf16_bytes=raw, quantized_bytes=packed)


def clear_model(model) -> None:
    for p in model.parameters():
        if hasattr(p, "_rlb_q"):
            del p._rlb_q
        if hasattr(p, "_rlb_q_bf16"):
            del p._rlb_q_bf16


def quantized_linear(x: torch.Tensor, qz, bias: Optional[torch.Tensor], residual: Optional[torch.Tensor], expanded=None) -> torch.Tensor:
    kind, q, s = qz
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if kind == "mxfp8":
        if x2.is_cuda:
            xb = x2 if x2.dtype == torch.bfloat16 else x2.to(torch.bfloat16)
            xq, xs = Q.quantize_mxfp8_blocked(xb.contiguous())   # scales land in the tensor core's layout directly
            y = Q.gemm_mxfp8(xq, xs, q, s)
        else:
            xq, xs = Q.quantize_mxfp8_ref(x2.to(torch.bfloat16))
            y = Q.dequantize_mxfp8(xq, xs).float() @ Q.dequantize_mxfp8(q, s).float().t()
    else:
        w = expanded if expanded is not None else Q.dequantize_fp8_blockwise(q, s)
        if x2.is_cuda:
            from rl_b200.ops import functional as F

            y = F.gemm(x2 if x2.dtype == torch.bfloat16 else x2.to(torch.bfloat16), w)
        else:
            y = x2.float() @ w.float().t()
    y = y.to(x.dtype)
    if bias is not None:
        y = y + bias
    y = y.reshape(*lead, y.shape[-1])
    return y if residual is None else y + residual
