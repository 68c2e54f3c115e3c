"""FP8 weight quantisation used by refit into FP8 engines: 128x128 block scales and MXFP8 (1x32 groups, E8M0 scales).

``quantize_fp8_blockwise`` follows ``cast_tensor_to_fp8_blockwise`` of the reference
(nemo_rl/models/generation/vllm/quantization/fp8.py:533-620): per-block amax, de-scale = amax / 448 (optionally rounded
up to a power of two), saturating cast to e4m3, ragged edges padded with the matrix's last element. ``quantize_mxfp8``
produces e4m3 data with one E8M0 scale byte per 32 consecutive elements of a row (scale = 2^ceil(log2(amax / 448)), so
nothing saturates). On a GPU both run as one native kernel; the torch forms below are the CPU path and the test oracle.
"""

from __future__ import annotations

import torch

from rl_b200.ops import lib as _L
from rl_b200.ops.lib import P, I, L, F as _F, call, ptr, register, stream_ptr, use_native

FP8_MAX = 448.0
E4M3 = torch.float8_e4m3fn

register("rlb_quant_fp8_block128", [P, L, P, L, P, I, I, I, _F, P])
register("rlb_quant_mxfp8", [P, L, P, L, P, L, I, I, P])
register("rlb_quant_mxfp8_blocked", [P, L, P, L, P, I, I, P])
register("rlb_dequant_fp8_block128", [P, L, P, P, L, I, I, P])
register("rlb_dequant_mxfp8", [P, L, P, L, P, L, I, I, P])


def _pow2_descale(descale: torch.Tensor):
    mant, ex = torch.frexp(descale)  # exact ceil(log2(x)): x = mant * 2^ex with mant in [0.5, 1)
    e = torch.where(mant == 0.5, ex - 1, ex).float().clamp(-127, 127) + 127
    e = torch.where(descale > 0, e, torch.zeros_like(e)).to(torch.uint8)
    ds = torch.where(e == 0, torch.ones_like(descale), torch.exp2(e.float() - 127))
    return ds, e


def quantize_fp8_blockwise_ref(w: torch.Tensor, block: int = 128, pow2: bool = False):
    R, C = w.shape
    pr, pc = (-R) % block, (-C) % block
    x = w.float()
    if pr or pc:
        x = torch.nn.functional.pad(x, (0, pc, 0, pr), value=float(x[-1, -1]))
    br, bc = x.shape[0] // block, x.shape[1] // block
    xb = x.reshape(br, block, bc, block).permute(0, 2, 1, 3)
    amax = xb.abs().amax(dim=(-1, -2))
    if pow2:
        ds, _ = _pow2_descale(amax / FP8_MAX)
        scale = 1.0 / ds
    else:
        scale = torch.where((amax == 0) | torch.isinf(amax), torch.ones_like(amax), FP8_MAX / amax)
        ds = 1.0 / scale
    q = (xb * scale[:, :, None, None]).clamp(-FP8_MAX, FP8_MAX).to(E4M3)
    q = q.permute(0, 2, 1, 3).reshape(x.shape)[:R, :C].contiguous()
    return q, ds


def quantize_fp8_blockwise(w: torch.Tensor, pow2: bool = False):
    """bf16 [R, C] -> (e4m3 [R, C], fp32 de-scale [ceil(R/128), ceil(C/128)]); ``w ~= q.float() * descale[block]``."""
    if not (use_native(w) and w.dtype == torch.bfloat16):
        return quantize_fp8_blockwise_ref(w, 128, pow2)
    R, C = w.shape
    w = w if w.stride(1) == 1 else w.contiguous()
    q = torch.empty((R, C), dtype=E4M3, device=w.device)
    ds = torch.empty(((R + 127) // 128, (C + 127) // 128), dtype=torch.float32, device=w.device)
    pad_abs = float(w[-1, -1].abs()) if (R % 128 or C % 128) else 0.0
    call("rlb_quant_fp8_block128", ptr(w), w.stride(0), ptr(q), q.stride(0), ptr(ds), R, C, int(pow2), pad_abs, stream_ptr())
    return q, ds


def dequantize_fp8_blockwise(q: torch.Tensor, descale: torch.Tensor) -> torch.Tensor:
    R, C = q.shape
    if use_native(q):
        out = torch.empty((R, C), dtype=torch.bfloat16, device=q.device)
        call("rlb_dequant_fp8_block128", ptr(q), q.stride(0), ptr(descale.contiguous()), ptr(out), out.stride(0), R, C, stream_ptr())
        return out
    ds = descale.repeat_interleave(128, 0)[:R].repeat_interleave(128, 1)[:, :C]
    return (q.float() * ds).to(torch.bfloat16)


def dequantize_fp8_blockwise_into(q: torch.Tensor, descale: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """Expands block-128 FP8 into an existing bf16 matrix (the engine's weight buffer keeps its address)."""
    R, C = q.shape
    assert out.shape == q.shape and out.dtype == torch.bfloat16 and out.stride(1) == 1
    if use_native(q):
        call("rlb_dequant_fp8_block128", ptr(q), q.stride(0), ptr(descale.contiguous()), ptr(out), out.stride(0), R, C, stream_ptr())
    else:
        out.copy_(dequantize_fp8_blockwise(q, descale))
    return out


def quantize_mxfp8_ref(w: torch.Tensor):
    R, C = w.shape
    assert C % 32 == 0
    x = w.float().reshape(R, C // 32, 32)
    amax = x.abs().amax(-1)
    ds, e = _pow2_descale(amax / FP8_MAX)
    q = (x / ds[..., None]).clamp(-FP8_MAX, FP8_MAX).to(E4M3).reshape(R, C)
    return q, e


def quantize_mxfp8(w: torch.Tensor):
    """bf16 [R, C] (C % 32 == 0) -> (e4m3 [R, C], uint8 E8M0 scales [R, C/32]); value = q * 2^(scale - 127)."""
    if not (use_native(w) and w.dtype == torch.bfloat16):
        return quantize_mxfp8_ref(w)
    R, C = w.shape
    w = w if w.stride(1) == 1 else w.contiguous()
    q = torch.empty((R, C), dtype=E4M3, device=w.device)
    sc = torch.empty((R, C // 32), dtype=torch.uint8, device=w.device)
    call("rlb_quant_mxfp8", ptr(w), w.stride(0), ptr(q), q.stride(0), ptr(sc), sc.stride(0), R, C, stream_ptr())
    return q, sc


def quantize_mxfp8_blocked(w: torch.Tensor):
    """bf16 [R, C] (C % 128 == 0, CUDA) -> (e4m3 [R, C], scales in the blocked layout of :func:`swizzle_mx_scales`), in one
    kernel: what the activation side of an MXFP8 linear needs on every call."""
    R, C = w.shape
    q = torch.empty((R, C), dtype=torch.float8_e4m3fn, device=w.device)
    sc = torch.empty((-(-R // 128), C // 128, 512), dtype=torch.uint8, device=w.device)
    call("rlb_quant_mxfp8_blocked", ptr(w), w.stride(0), ptr(q), q.stride(0), ptr(sc), R, C, stream_ptr())
    return q, sc


def dequantize_mxfp8(q: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    R, C = q.shape
    if use_native(q):
        out = torch.empty((R, C), dtype=torch.bfloat16, device=q.device)
        call("rlb_dequant_mxfp8", ptr(q), q.stride(0), ptr(scales), scales.stride(0), ptr(out), out.stride(0), R, C, stream_ptr())
        return out
    ds = torch.where(scales == 0, torch.ones((), dtype=torch.float32), torch.exp2(scales.float() - 127))
    return (q.float().reshape(R, C // 32, 32) * ds[..., None]).reshape(R, C).to(torch.bfloat16)


# --------------------------------------------------------------------------------------------- MXFP8 GEMM
register("rlb_gemm_mxfp8", [P, L, P, L, P, P, P, L, I, I, I, P, P])


def swizzle_mx_scales(scales: torch.Tensor) -> torch.Tensor:
    """Row-major E8M0 scales [R, K/32] -> the blocked layout the tensor core reads: [ceil(R/128), K/128, 512] bytes, where
    row r of a 128-row block and 32-wide K group j of a 128-wide K block sit at byte (r % 32) * 16 + (r // 32) * 4 + j.
    Rows beyond R are filled with scale byte 0."""
    R, G = scales.shape
    assert G % 4 == 0, "K must be a multiple of 128"
    Rb = -(-R // 128)
    s = torch.zeros((Rb * 128, G), dtype=torch.uint8, device=scales.device)
    s[:R] = scales
    s = s.view(Rb, 4, 32, G // 4, 4).permute(0, 3, 2, 1, 4)  # [Rb, Kb, r % 32, r // 32, j]
    return s.reshape(Rb, G // 4, 512).contiguous()


def gemm_mxfp8(a_q: torch.Tensor, a_sf: torch.Tensor, b_q: torch.Tensor, b_sf: torch.Tensor) -> torch.Tensor:
    """C [M, N] bf16 = dequant(A) @ dequant(B)^T for MXFP8 operands: ``a_q`` [M, K] / ``b_q`` [N, K] e4m3 and their scales in
    the blocked layout of :func:`swizzle_mx_scales`. The scales are applied by the tensor core (block-scaled MMA)."""
    M, K = a_q.shape
    N = b_q.shape[0]
    if not use_native(a_q):
        raise RuntimeError("the MXFP8 GEMM needs the native library on a GPU")
    out = torch.empty((M, N), dtype=torch.bfloat16, device=a_q.device)
    call("rlb_gemm_mxfp8", ptr(a_q), a_q.stride(0), ptr(b_q), b_q.stride(0), ptr(a_sf), ptr(b_sf), ptr(out), out.stride(0), M, N, K,
         ptr(_L.status_word(a_q.device)), stream_ptr())
    return out
