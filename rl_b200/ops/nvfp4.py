"""NVFP4 (block-16 E2M1 values, one E4M3 scale per block, one fp32 scale per tensor) and per-tensor FP8 quantisation:
exact pack / unpack and the "fake" (quantise-dequantise) forms with a straight-through gradient that quantisation-aware
training uses. The format is Blackwell's native 4-bit tensor-core input (``tcgen05.mma.kind::mxf4nvf4``); the reference
reaches it through ModelOpt's quantizers (nemo_rl/modelopt/utils.py: group size 16, ``weight_scale`` / ``weight_scale_2`` /
``input_scale`` tensors).

Value of an element: ``e2m1 * e4m3_block_scale * tensor_scale`` with ``tensor_scale = amax * fp32(1 / (6 * 448))`` so that the largest
block scale is representable, ``e4m3_block_scale = round_e4m3(block_amax / 6 / tensor_scale)`` and ``e2m1`` the nearest of
{0, 0.5, 1, 1.5, 2, 3, 4, 6} (ties to the even mantissa) with a sign.
"""

from __future__ import annotations

from typing import Optional

import torch

from rl_b200.ops.lib import I, L, P, register

register("rlb_fake_quant_nvfp4", [P, P, P, L, L, I, I, P])
register("rlb_quant_nvfp4", [P, P, P, P, L, L, I, I, P])

E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
E2M1_MAX, E4M3_MAX, BLOCK = 6.0, 448.0, 16
# midpoints between neighbouring values; a tie goes to the value with the even mantissa (0, 1, 2, 4), which for the midpoints
# 0.75, 1.75 and 3.5 is the upper neighbour: those thresholds sit one ulp lower so that ``<=`` sends the tie up
_BOUNDS = (0.25, 0.7499999, 1.25, 1.7499999, 2.5, 3.4999998, 5.0)


def _tables(device):
    return (torch.tensor(E2M1_VALUES, dtype=torch.float32, device=device), torch.tensor(_BOUNDS, dtype=torch.float32, device=device))


# fp32 reciprocals of 6 * 448 and of 6, spelled out so that this statement and the kernel multiply by the same bits (a
# division by a Python scalar is evaluated differently for 0-dim and n-dim tensors)
_INV_RANGE, _INV_E2M1_MAX = float.fromhex("0x1.861862p-12"), float.fromhex("0x1.555556p-3")


def tensor_scale(amax: torch.Tensor) -> torch.Tensor:
    return (amax.float() * _INV_RANGE).clamp(min=1e-30)


def _block_view(x: torch.Tensor):
    assert x.shape[-1] % BLOCK == 0, "the last dimension must be a multiple of 16"
    return x.float().reshape(*x.shape[:-1], x.shape[-1] // BLOCK, BLOCK)


def _codes_and_scales(x: torch.Tensor, amax: Optional[torch.Tensor]):
    """(sign-magnitude codes 0..15 [.., n/16, 16], E4M3 block scales as fp32 [.., n/16], tensor scale)."""
    xb = _block_view(x)
    s2 = tensor_scale(xb.abs().amax() if amax is None else amax)      # scalar, or [.., 1, 1] against the [.., rows, blocks] scales
    want = xb.abs().amax(-1) * _INV_E2M1_MAX / s2
    sb = want.clamp(max=E4M3_MAX).to(torch.float8_e4m3fn).float()            # what the 8-bit scale can hold
    step = (sb * s2).unsqueeze(-1)
    mag = torch.where(step > 0, xb.abs() / step.clamp(min=1e-30), torch.zeros_like(xb)).clamp(max=E2M1_MAX)
    vals, bounds = _tables(x.device)
    idx = torch.bucketize(mag, bounds, right=False)                          # 0..7
    return idx + (xb < 0).to(idx.dtype) * 8, sb, s2


def quantize_nvfp4(x: torch.Tensor, amax: Optional[torch.Tensor] = None):
    """-> (packed uint8 [.., n/2] (element 2i in the low nibble), block scales float8_e4m3fn [.., n/16], tensor scale fp32)."""
    g = _native_groups(x, amax)
    if g is not None and g[0].numel() == 1:
        from rl_b200.ops import lib as _L

        packed = torch.empty((*x.shape[:-1], x.shape[-1] // 2), dtype=torch.uint8, device=x.device)
        sb8 = torch.empty((*x.shape[:-1], x.shape[-1] // BLOCK), dtype=torch.float8_e4m3fn, device=x.device)
        _L.call("rlb_quant_nvfp4", _L.ptr(x), _L.ptr(packed), _L.ptr(sb8), _L.ptr(g[0]), g[1], g[2], x.shape[-1],
                0 if x.dtype == torch.bfloat16 else 1, _L.stream_ptr())
        return packed, sb8, tensor_scale(g[0]).reshape(())
    codes, sb, s2 = _codes_and_scales(x, amax)
    c = codes.reshape(*x.shape[:-1], x.shape[-1] // 2, 2).to(torch.uint8)
    return (c[..., 0] | (c[..., 1] << 4)), sb.to(torch.float8_e4m3fn), s2.reshape(())


def dequantize_nvfp4(packed: torch.Tensor, block_scales: torch.Tensor, s2: torch.Tensor, dtype=torch.float32) -> torch.Tensor:
    vals, _ = _tables(packed.device)
    lo, hi = (packed & 0xF).long(), (packed >> 4).long()
    codes = torch.stack([lo, hi], dim=-1).reshape(*packed.shape[:-1], packed.shape[-1] * 2)
    v = vals[codes & 7] * torch.where(codes >= 8, -1.0, 1.0)
    v = v.reshape(*v.shape[:-1], v.shape[-1] // BLOCK, BLOCK) * (block_scales.float() * s2.float()).unsqueeze(-1)
    return v.reshape(*packed.shape[:-1], packed.shape[-1] * 2).to(dtype)


def _native_groups(x: torch.Tensor, amax: Optional[torch.Tensor]):
    """(amax as a flat fp32 device tensor, rows per entry, rows) when the native kernels cover this call, else None."""
    from rl_b200.ops import lib as _L

    if not (_L.use_native(x) and _L.available() and x.dtype in (torch.bfloat16, torch.float32) and x.dim() >= 2
            and x.is_contiguous() and x.shape[-1] % BLOCK == 0 and x.numel() > 0 and x.data_ptr() % 16 == 0):
        return None
    R = x.numel() // x.shape[-1]
    if amax is None:
        return x.detach().abs().amax().float().reshape(1), R, R
    a = amax.detach().float().to(x.device)
    if a.numel() == 1:
        return a.reshape(1).contiguous(), R, R
    if x.dim() == 3 and a.numel() == x.shape[0]:
        return a.reshape(-1).contiguous(), x.shape[1], R
    return None


def _fake_nvfp4(x: torch.Tensor, amax: Optional[torch.Tensor]) -> torch.Tensor:
    g = _native_groups(x, amax)
    if g is not None:     # one streaming kernel (csrc/nvfp4.cu), the same bits as the statement below
        from rl_b200.ops import lib as _L

        out = torch.empty_like(x)
        _L.call("rlb_fake_quant_nvfp4", _L.ptr(x), _L.ptr(out), _L.ptr(g[0]), g[1], g[2], x.shape[-1], 0 if x.dtype == torch.bfloat16 else 1,
                _L.stream_ptr())
        return out
    codes, sb, s2 = _codes_and_scales(x, amax)
    vals, _ = _tables(x.device)
    v = vals[codes & 7] * torch.where(codes >= 8, -1.0, 1.0) * (sb * s2).unsqueeze(-1)
    return v.reshape(x.shape).to(x.dtype)


def _fake_fp8(x: torch.Tensor, amax: Optional[torch.Tensor]) -> torch.Tensor:
    a = (x.abs().amax() if amax is None else amax).float().clamp(min=1e-30)
    s = a / E4M3_MAX
    return ((x.float() / s).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).float() * s).to(x.dtype)


class _StraightThrough(torch.autograd.Function):
    """Quantise-dequantise in the forward pass; the gradient passes unchanged (values beyond a static range get none)."""

    @staticmethod
    def forward(ctx, x, amax, kind, clip):
        ctx.clipped = amax is not None and clip
        if ctx.clipped:
            ctx.save_for_backward(x.abs() <= amax)
        return (_fake_nvfp4 if kind == "nvfp4" else _fake_fp8)(x, amax)

    @staticmethod
    def backward(ctx, g):
        if ctx.clipped:
            (inside,) = ctx.saved_tensors
            g = g * inside
        return g, None, None, None


def fake_quant(x: torch.Tensor, kind: str = "nvfp4", amax: Optional[torch.Tensor] = None, clip: bool = True) -> torch.Tensor:
    """``kind``: "nvfp4" (block-16 E2M1) or "fp8" (per-tensor E4M3). ``amax``: the tensor-level range (None: this tensor's own
    maximum, i.e. dynamic); a scalar, or one value per leading index (e.g. [E, 1, 1] for stacked expert matrices, each a tensor
    of its own). ``clip``: values beyond a given range get no gradient."""
    if kind not in ("nvfp4", "fp8"):
        raise ValueError(f"unknown quantisation kind {kind!r}")
    if x.requires_grad and torch.is_grad_enabled():
        return _StraightThrough.apply(x, amax, kind, clip)
    return (_fake_nvfp4 if kind == "nvfp4" else _fake_fp8)(x, amax)
