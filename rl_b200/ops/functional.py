"""Tensor-level operators.

Each operator has two bodies: the native sm_100a kernel (CUDA tensors) and a plain PyTorch restatement
(CPU tensors) that serves as the numerical oracle in tests and as the CPU/gloo execution path. Autograd
is wired by hand so that the backward pass also runs on the native kernels.
"""

from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as tF

from . import lib as _L
from .lib import call, ptr, stream_ptr, use_native

BF16 = torch.bfloat16
SKINNY_MAX_M = 256  # batches up to this many rows take the weight-streaming GEMM


# --------------------------------------------------------------------------------------- GEMM
def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    a_mn: bool = False,
    b_mn: bool = False,
    out: Optional[torch.Tensor] = None,
    out_dtype: torch.dtype = BF16,
    accumulate: bool = False,
    bias: Optional[torch.Tensor] = None,
    residual: Optional[torch.Tensor] = None,
    max_ctas: int = 0,
) -> torch.Tensor:
    """C[M,N] = op(A) @ op(B)^T. ``a`` is [M,K] (or [K,M] when ``a_mn``), ``b`` is [N,K] (or [K,N] when ``b_mn``).

    Rows may be strided (views into wider buffers) as long as the last dimension is contiguous.
    """
    assert a.dim() == 2 and b.dim() == 2
    M, K = (a.shape[1], a.shape[0]) if a_mn else a.shape
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else b.shape
    assert K == Kb, f"inner dimensions differ: {K} vs {Kb}"
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
        assert not accumulate
    if not use_native(a):
        A = a.t() if a_mn else a
        B = b if b_mn else b.t()
        res = A.float() @ B.float()
        if bias is not None:
            res = res + bias.float()
        if residual is not None:
            res = res + residual.float()
        if accumulate:
            res = res + out.float()
        out.copy_(res.to(out.dtype))
        return out
    assert a.dtype == BF16 and b.dtype == BF16, "native GEMM takes bf16 operands"
    if a.stride(1) != 1:
        a = a.contiguous()
    if b.stride(1) != 1:
        b = b.contiguous()
    assert out.stride(1) == 1 and out.dtype in (BF16, torch.float32)
    if bias is not None:
        bias = bias.float().contiguous()
    if M <= SKINNY_MAX_M and not a_mn and not b_mn and not accumulate and max_ctas == 0 and K >= 256:
        # decode-sized batches: weight-streaming kernel with cluster split-K
        call("rlb_gemm_skinny", ptr(a), ptr(b), ptr(out), M, N, K, a.stride(0), b.stride(0), out.stride(0),
             int(out.dtype == torch.float32), ptr(bias), ptr(residual), residual.stride(0) if residual is not None else 0,
             0, ptr(_L.status_word(a.device)), stream_ptr())
        return out
    call(
        "rlb_gemm_bf16", ptr(a), ptr(b), ptr(out), M, N, K, a.stride(0), b.stride(0), out.stride(0),
        int(a_mn), int(b_mn), int(out.dtype == torch.float32), int(accumulate), ptr(bias),
        ptr(residual), residual.stride(0) if residual is not None else 0,
        ptr(_L.status_word(a.device)), max_ctas, stream_ptr(),
    )
    return out


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, residual):
        ctx.save_for_backward(x, w)
        ctx.has_bias = bias is not None
        x2 = x.reshape(-1, x.shape[-1])
        r2 = None
        if residual is not None:
            r2 = residual.reshape(-1, residual.shape[-1])
            assert r2.dtype == BF16 and r2.stride(-1) == 1
        # the result is allocated in its final shape so that the returned tensor is not a view (in-place consumers
        # such as RoPE may then modify it under autograd)
        y = torch.empty((*x.shape[:-1], w.shape[0]), dtype=x.dtype, device=x.device)
        gemm(x2, w, bias=bias, residual=r2, out=y.view(-1, w.shape[0]))
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        x2 = x.reshape(-1, x.shape[-1])
        if dy2.stride(-1) != 1:
            dy2 = dy2.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, b_mn=True, out_dtype=x.dtype).view_as(x)
        if ctx.needs_input_grad[1]:
            main_grad = getattr(w, "main_grad", None)
            if main_grad is not None:
                # weight gradient accumulates straight into the (bf16 or fp32) gradient buffer
                gemm(dy2, x2, a_mn=True, b_mn=True, out=main_grad, accumulate=True)
                dw = None
            else:
                dw = gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=w.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0)
            bias_grad = getattr(ctx, "bias_main_grad", None)
        dres = dy if ctx.needs_input_grad[3] else None
        return dx, dw, db, dres


# --------------------------------------------------------------------------------------- MXFP8 training linear
class Fp8Training:
    """Process-wide switch for block-scaled FP8 training of the linear layers (``policy.fp8_cfg`` /
    ``megatron_cfg.fp8_cfg`` with ``fp8_recipe: mxfp8``; nemo_rl/models/policy/__init__.py:290-306,
    nemo_rl/models/megatron/setup.py:1131-1178). Master weights, gradients and the optimizer stay bf16 / fp32; only the
    three GEMMs of a linear layer (forward, input gradient, weight gradient) take MXFP8 operands (e4m3 with one E8M0
    scale per 32 elements along the contraction dimension), each quantised along the dimension that GEMM contracts.
    ``epoch`` must be advanced whenever the weights change (after an optimizer step) so that cached weight copies are
    re-quantised."""

    enabled = False
    epoch = 0
    stats = dict(fwd=0, dgrad=0, wgrad=0, weight_quantisations=0)

    @classmethod
    def configure(cls, cfg: Optional[dict]) -> bool:
        c = cfg or {}
        cls.enabled = bool(c.get("enabled")) and c.get("fp8_recipe", "mxfp8") in ("mxfp8", "blockwise")
        return cls.enabled

    @classmethod
    def weights_changed(cls) -> None:
        cls.epoch += 1


def _mx_fake(x: torch.Tensor) -> torch.Tensor:
    """CPU statement of MXFP8 rounding along the last dimension (quantise, de-quantise)."""
    from . import quant as Q

    R, C = x.shape
    pad = (-C) % 32
    xp = tF.pad(x.float(), (0, pad)) if pad else x.float()
    q, e = Q.quantize_mxfp8_ref(xp.to(torch.bfloat16))
    return Q.dequantize_mxfp8(q, e).float()[:, :C]


def _mx_operand(t: torch.Tensor):
    """bf16 [R, C] -> MXFP8 operand quantised along C; rows and columns are zero-padded to multiples of 128."""
    from . import quant as Q

    R, C = t.shape
    pr, pc = (-R) % 128, (-C) % 128
    if pr or pc:
        t = tF.pad(t, (0, pc, 0, pr))
    return Q.quantize_mxfp8_blocked(t.contiguous())


def _mx_gemm(a: torch.Tensor, b: torch.Tensor, a_op=None, b_op=None) -> torch.Tensor:
    """a [M, K] @ b[N, K]^T with both operands rounded to MXFP8 along K (block-scaled tensor-core GEMM on the GPU)."""
    from . import quant as Q

    M, N = a.shape[0], b.shape[0]
    if not use_native(a):
        return (_mx_fake(a) @ _mx_fake(b).t()).to(a.dtype)
    aq, asf = a_op if a_op is not None else _mx_operand(a)
    bq, bsf = b_op if b_op is not None else _mx_operand(b)
    return Q.gemm_mxfp8(aq, asf, bq, bsf)[:M, :N]


def _mx_weight(w: torch.Tensor, transposed: bool):
    """Cached MXFP8 copy of a weight (or of its transpose), refreshed when ``Fp8Training.epoch`` moves."""
    key = "_rlb_mx_t" if transposed else "_rlb_mx"
    cur = getattr(w, key, None)
    if cur is not None and cur[0] == Fp8Training.epoch:
        return cur[1]
    op = _mx_operand((w.detach().t() if transposed else w.detach()).contiguous())
    setattr(w, key, (Fp8Training.epoch, op))
    Fp8Training.stats["weight_quantisations"] += 1
    return op


class _MXLinear(torch.autograd.Function):
    """y = x W^T with MXFP8 GEMMs in forward, input gradient and weight gradient (bf16 master weight, fp32 / bf16
    gradient accumulation as in the bf16 path)."""

    @staticmethod
    def forward(ctx, x, w, bias, residual):
        x2 = x.reshape(-1, x.shape[-1])
        native = use_native(x2)
        y = _mx_gemm(x2, w, b_op=_mx_weight(w, False) if native else None)
        Fp8Training.stats["fwd"] += 1
        if bias is not None:
            y = y + bias.to(y.dtype)
        y = y.reshape(*x.shape[:-1], w.shape[0])
        if residual is not None:
            y = y + residual
        ctx.save_for_backward(x, w)
        ctx.has_bias = bias is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        x2 = x.reshape(-1, x.shape[-1])
        native = use_native(dy2)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            # dX [M, K] = dY [M, N] W [N, K]: contraction over N, so W is quantised along N (its transpose along the rows)
            dx = _mx_gemm(dy2, w.t().contiguous() if not native else w, b_op=_mx_weight(w, True) if native else None)
            if not native:
                pass
            dx = dx.reshape(x.shape)
            Fp8Training.stats["dgrad"] += 1
        if ctx.needs_input_grad[1]:
            # dW [N, K] = dY^T [N, M] X [M, K]: contraction over the tokens
            g = _mx_gemm(dy2.t().contiguous(), x2.t().contiguous())
            Fp8Training.stats["wgrad"] += 1
            main_grad = getattr(w, "main_grad", None)
            if main_grad is not None:
                main_grad.add_(g.to(main_grad.dtype))
            else:
                dw = g.to(w.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0)
        dres = dy if ctx.needs_input_grad[3] else None
        return dx, dw, db, dres


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
           residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x @ w^T (+ bias) (+ residual); w is [out_features, in_features] as in ``nn.Linear``.

    ``residual`` (same shape as y) is added inside the GEMM epilogue, which saves one read-modify-write pass over
    the residual stream per projection."""
    qat = getattr(w, "_rlb_qat", None)
    if qat is not None:      # quantisation-aware training: quantise-dequantise the operands, then the usual product
        from rl_b200.policy.qat import QatState

        if QatState.enabled:
            x, w = qat.q_input(x), qat.q_weight(w)
    qz = getattr(w, "_rlb_q", None)
    if qz is not None and not torch.is_grad_enabled():
        from rl_b200.engine import quantized as _qz   # low-precision rollout: only inside the engine's generation phase

        if _qz.is_active():
            return _qz.quantized_linear(x, qz, bias, residual, getattr(w, "_rlb_q_bf16", None))
    if Fp8Training.enabled and torch.is_grad_enabled() and w.dim() == 2 and w.shape[0] % 16 == 0 and w.shape[1] % 32 == 0 \
            and w.requires_grad and not getattr(w, "_rlb_keep_bf16", False):
        return _MXLinear.apply(x, w, bias, residual)
    if not use_native(x):
        y = tF.linear(x, w, bias)
        return y if residual is None else y + residual
    return _Linear.apply(x, w, bias, residual)


# --------------------------------------------------------------------------------------- RMSNorm
def _rmsnorm_ref(x, w, eps):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    return y.to(x.dtype)


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        d = x.shape[-1]
        x2 = x.reshape(-1, d)
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        rows = x2.shape[0]
        y = torch.empty((rows, d), dtype=x.dtype, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        call("rlb_rmsnorm_fwd", ptr(x2), None, ptr(w), ptr(y), None, ptr(rstd), rows, d, x2.stride(0), d, eps, stream_ptr())
        ctx.save_for_backward(x2, w, rstd)
        ctx.shape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w, rstd = ctx.saved_tensors
        rows, d = x2.shape
        dy2 = dy.reshape(rows, d)
        if dy2.stride(-1) != 1:
            dy2 = dy2.contiguous()
        dx = torch.empty((rows, d), dtype=x2.dtype, device=x2.device)
        parts = _L.lib().rlb_rmsnorm_bwd_parts(rows)
        partial = torch.empty((parts, d), dtype=torch.float32, device=x2.device)
        main_grad = getattr(w, "main_grad", None)
        if main_grad is not None:
            f32 = main_grad if main_grad.dtype == torch.float32 else None
            b16 = main_grad if main_grad.dtype == BF16 else None
            call("rlb_rmsnorm_bwd", ptr(dy2), ptr(x2), ptr(w), ptr(rstd), ptr(dx), ptr(partial), ptr(f32), ptr(b16), 1,
                 rows, d, x2.stride(0), dy2.stride(0), 0, stream_ptr())
            dw = None
        else:
            dw32 = torch.empty(d, dtype=torch.float32, device=x2.device)
            call("rlb_rmsnorm_bwd", ptr(dy2), ptr(x2), ptr(w), ptr(rstd), ptr(dx), ptr(partial), ptr(dw32), None, 0,
                 rows, d, x2.stride(0), dy2.stride(0), 0, stream_ptr())
            dw = dw32.to(w.dtype)
        return dx.view(ctx.shape), dw, None


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    if not use_native(x):
        return _rmsnorm_ref(x, w, eps)
    return _RMSNorm.apply(x, w, eps)


def rmsnorm_residual_(x: torch.Tensor, residual: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """Inference-only fusion: residual += x (in place), returns rmsnorm(residual)."""
    if not use_native(x):
        residual.add_(x)
        return _rmsnorm_ref(residual, w, eps)
    d = x.shape[-1]
    x2 = x.reshape(-1, d)
    r2 = residual.view(-1, d)
    y = torch.empty_like(r2)
    call("rlb_rmsnorm_fwd", ptr(x2), ptr(r2), ptr(w), ptr(y), ptr(r2), None, x2.shape[0], d, x2.stride(0), d, eps, stream_ptr())
    return y.view(residual.shape)


# --------------------------------------------------------------------------------------- per-head RMSNorm (Qwen3)
class _HeadRMSNorm(torch.autograd.Function):
    """Normalises ``heads`` consecutive head vectors of width D starting at column ``col0`` of each row of a
    [T, C] buffer; the other columns are passed through untouched (a copy)."""

    @staticmethod
    def forward(ctx, buf, w, col0, heads, D, eps):
        T = buf.shape[0]
        out = buf.clone()
        rstd = torch.empty(T * heads, dtype=torch.float32, device=buf.device)
        src = buf[:, col0:]
        dst = out[:, col0:]
        call("rlb_head_rmsnorm_fwd", ptr(src), ptr(w), ptr(dst), ptr(rstd), T, heads, D, buf.stride(0), out.stride(0), eps, stream_ptr())
        ctx.save_for_backward(buf, w, rstd)
        ctx.meta = (col0, heads, D)
        return out

    @staticmethod
    def backward(ctx, dout):
        buf, w, rstd = ctx.saved_tensors
        col0, heads, D = ctx.meta
        T = buf.shape[0]
        dout = dout.contiguous()
        dbuf = dout.clone()
        dw = torch.zeros(D, dtype=torch.float32, device=buf.device)
        call("rlb_head_rmsnorm_bwd", ptr(dout[:, col0:]), ptr(buf[:, col0:]), ptr(w), ptr(rstd), ptr(dbuf[:, col0:]), ptr(dw),
             T, heads, D, buf.stride(0), dout.stride(0), dbuf.stride(0), stream_ptr())
        main_grad = getattr(w, "main_grad", None)
        if main_grad is not None:
            main_grad.add_(dw.to(main_grad.dtype))
            return dbuf, None, None, None, None, None
        return dbuf, dw.to(w.dtype), None, None, None, None


def head_rmsnorm(buf: torch.Tensor, w: torch.Tensor, col0: int, heads: int, D: int, eps: float) -> torch.Tensor:
    if not use_native(buf):
        T = buf.shape[0]
        seg = buf[:, col0 : col0 + heads * D].reshape(T, heads, D)
        normed = _rmsnorm_ref(seg, w, eps).reshape(T, heads * D)
        return torch.cat([buf[:, :col0], normed, buf[:, col0 + heads * D :]], dim=1)
    return _HeadRMSNorm.apply(buf, w, col0, heads, D, eps)


# --------------------------------------------------------------------------------------- RoPE
def _rope_ref(x, positions, inv_freq, heads, D, sign=1.0):
    T = x.shape[0]
    seg = x[:, : heads * D].reshape(T, heads, D).float()
    ang = positions.float()[:, None] * inv_freq.float()[None, :]  # [T, D/2]
    cos, sin = ang.cos()[:, None, :], (ang.sin() * sign)[:, None, :]
    lo, hi = seg[..., : D // 2], seg[..., D // 2 :]
    out = torch.cat([lo * cos - hi * sin, hi * cos + lo * sin], dim=-1).reshape(T, heads * D)
    return torch.cat([out.to(x.dtype), x[:, heads * D :]], dim=1)


class _RopeInplace(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, positions, inv_freq, heads, D):
        call("rlb_rope", ptr(x), ptr(positions), ptr(inv_freq), x.shape[0], heads, D, x.stride(0), 0, stream_ptr())
        ctx.mark_dirty(x)
        ctx.save_for_backward(positions, inv_freq)
        ctx.meta = (heads, D)
        return x

    @staticmethod
    def backward(ctx, dy):
        positions, inv_freq = ctx.saved_tensors
        heads, D = ctx.meta
        dy = dy.contiguous() if dy.stride(-1) != 1 else dy
        dx = dy.clone()
        call("rlb_rope", ptr(dx), ptr(positions), ptr(inv_freq), dx.shape[0], heads, D, dx.stride(0), 1, stream_ptr())
        return dx, None, None, None, None


def rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, heads: int, D: int) -> torch.Tensor:
    """Rotates the first ``heads`` head vectors (width D, HF rotate_half convention) of each row of ``x`` [T, C].

    With a fused [q | k | v] projection output, ``heads = Hq + Hkv`` rotates q and k in one launch. On CUDA the
    rotation is in place (and the returned tensor is ``x``).
    """
    if not use_native(x):
        return _rope_ref(x, positions, inv_freq, heads, D)
    positions = positions.to(torch.int32)
    if torch.is_grad_enabled() and x.requires_grad:
        return _RopeInplace.apply(x, positions, inv_freq, heads, D)
    call("rlb_rope", ptr(x), ptr(positions), ptr(inv_freq), x.shape[0], heads, D, x.stride(0), 0, stream_ptr())
    return x


# --------------------------------------------------------------------------------------- SwiGLU
class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        F2 = gu.shape[-1]
        g2 = gu.reshape(-1, F2)
        y = torch.empty((g2.shape[0], F2 // 2), dtype=gu.dtype, device=gu.device)
        call("rlb_swiglu_fwd", ptr(g2), ptr(y), g2.shape[0], F2 // 2, stream_ptr())
        ctx.save_for_backward(g2)
        ctx.shape = gu.shape
        return y.view(*gu.shape[:-1], F2 // 2)

    @staticmethod
    def backward(ctx, dy):
        (g2,) = ctx.saved_tensors
        F = g2.shape[1] // 2
        dy2 = dy.reshape(-1, F).contiguous()
        dgu = torch.empty_like(g2)
        call("rlb_swiglu_bwd", ptr(dy2), ptr(g2), ptr(dgu), g2.shape[0], F, stream_ptr())
        return dgu.view(ctx.shape)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up for a fused [..., 2F] projection laid out as [gate | up]."""
    if not use_native(gate_up):
        g, u = gate_up.chunk(2, dim=-1)
        return (tF.silu(g.float()) * u.float()).to(gate_up.dtype)
    return _SwiGLU.apply(gate_up.contiguous())


def gated_act(gate_up: torch.Tensor, act: str = "silu") -> torch.Tensor:
    """act(gate) * up for a fused [..., 2F] projection: ``silu`` (SwiGLU, native kernel) or ``gelu_pytorch_tanh`` (GeGLU)."""
    if act == "silu":
        return swiglu(gate_up)
    g, u = gate_up.chunk(2, dim=-1)
    if act in ("gelu_pytorch_tanh", "gelu_tanh"):
        return (tF.gelu(g.float(), approximate="tanh") * u.float()).to(gate_up.dtype)
    if act == "gelu":
        return (tF.gelu(g.float()) * u.float()).to(gate_up.dtype)
    raise ValueError(f"unknown gate activation '{act}'")


def plain_act(x: torch.Tensor, act: str = "relu2") -> torch.Tensor:
    """Activation of a non-gated MLP: ``relu2`` (squared ReLU, Nemotron-H), ``silu``, ``gelu``, ``relu``."""
    if act == "relu2":
        return torch.relu(x).square()
    if act == "silu":
        return tF.silu(x)
    if act == "relu":
        return torch.relu(x)
    if act in ("gelu", "gelu_pytorch_tanh", "gelu_tanh"):
        return tF.gelu(x, approximate="none" if act == "gelu" else "tanh")
    raise ValueError(f"unknown activation '{act}'")


# --------------------------------------------------------------------------------------- embedding
class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table):
        flat = ids.reshape(-1).to(torch.int32)
        out = torch.empty((flat.numel(), table.shape[1]), dtype=table.dtype, device=table.device)
        call("rlb_embedding_fwd", ptr(flat), ptr(table), ptr(out), flat.numel(), table.shape[1], table.shape[0], stream_ptr())
        ctx.save_for_backward(flat)
        ctx.table = table
        return out.view(*ids.shape, table.shape[1])

    @staticmethod
    def backward(ctx, dy):
        (flat,) = ctx.saved_tensors
        table = ctx.table
        dy2 = dy.reshape(-1, table.shape[1]).contiguous()
        main_grad = getattr(table, "main_grad", None)
        if main_grad is not None and main_grad.dtype == torch.float32:
            call("rlb_embedding_bwd", ptr(flat), ptr(dy2), ptr(main_grad), flat.numel(), table.shape[1], table.shape[0], stream_ptr())
            return None, None
        g = torch.zeros(table.shape, dtype=torch.float32, device=table.device)
        call("rlb_embedding_bwd", ptr(flat), ptr(dy2), ptr(g), flat.numel(), table.shape[1], table.shape[0], stream_ptr())
        if main_grad is not None:
            main_grad.add_(g.to(main_grad.dtype))
            return None, None
        return None, g.to(table.dtype)


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    if not use_native(table):
        return tF.embedding(ids, table)
    return _Embedding.apply(ids, table)


# --------------------------------------------------------------------------------------- attention (varlen, causal, GQA)
def _attention_ref(qkv, cu_seqlens, Hq, Hkv, D, scale, window: int = 0):
    """``window`` > 0: a query sees only the last ``window`` keys up to and including itself (sliding-window layers)."""
    T = qkv.shape[0]
    q = qkv[:, : Hq * D].reshape(T, Hq, D)
    k = qkv[:, Hq * D : (Hq + Hkv) * D].reshape(T, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D :].reshape(T, Hkv, D)
    out = torch.empty((T, Hq, D), dtype=qkv.dtype, device=qkv.device)
    cu = cu_seqlens.tolist()
    g = Hq // Hkv
    for s, e in zip(cu[:-1], cu[1:]):
        if e <= s:
            continue
        qs = q[s:e].transpose(0, 1).unsqueeze(0)
        ks = k[s:e].transpose(0, 1).unsqueeze(0)
        vs = v[s:e].transpose(0, 1).unsqueeze(0)
        n = e - s
        if window and n > window:
            i = torch.arange(n, device=qkv.device)
            band = (i[None, :] <= i[:, None]) & (i[None, :] > i[:, None] - window)
            o = tF.scaled_dot_product_attention(qs, ks, vs, attn_mask=band, scale=scale, enable_gqa=g > 1)
        else:
            o = tF.scaled_dot_product_attention(qs, ks, vs, is_causal=True, scale=scale, enable_gqa=g > 1)
        out[s:e] = o[0].transpose(0, 1)
    return out.reshape(T, Hq * D)


_attn_impl = None


def set_attention_impl(fn) -> None:
    """Installs the native varlen attention (set by :mod:`rl_b200.ops.attention` when its kernels are present)."""
    global _attn_impl
    _attn_impl = fn


def attention_varlen(qkv: torch.Tensor, cu_seqlens: torch.Tensor, max_seqlen: int, Hq: int, Hkv: int, D: int,
                     scale: Optional[float] = None, window: int = 0) -> torch.Tensor:
    """Causal self-attention over packed sequences. ``qkv`` is the fused projection output [T, (Hq+2Hkv)*D] (after
    RoPE); ``cu_seqlens`` [B+1] int32 are the packed sequence boundaries. Returns [T, Hq*D]. ``window`` > 0 restricts every
    query to its last ``window`` keys (the native kernels have no window: sequences longer than it take the PyTorch path)."""
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if use_native(qkv) and _attn_impl is not None and not (window and max_seqlen > window):
        return _attn_impl(qkv, cu_seqlens, max_seqlen, Hq, Hkv, D, scale)
    return _attention_ref(qkv, cu_seqlens, Hq, Hkv, D, scale, window)


# --------------------------------------------------------------------------------------- fused lm_head -> logprob / entropy
def _lm_head_ref(h, w, targets, inv_temp, want_entropy):
    z = (h.float() @ w.float().t()) * inv_temp
    lse = torch.logsumexp(z, dim=-1)
    logp = z.gather(-1, targets.long().unsqueeze(-1)).squeeze(-1) - lse
    ent = None
    if want_entropy:
        p = torch.softmax(z, dim=-1)
        ent = lse - (p * z).sum(-1)
    return logp, ent


class _LMHeadLogprob(torch.autograd.Function):
    """log p(target) (and entropy) of softmax(h W^T / T) without materialising the [T, V] logits in forward.
    Backward recomputes the logits tile by tile into a bf16 dZ chunk and feeds the dH / dW GEMMs."""

    CHUNK = 8192

    @staticmethod
    def forward(ctx, h, w, targets, inv_temp, want_entropy):
        M, K = h.shape
        N = w.shape[0]
        dev = h.device
        parts = _L.lib().rlb_gemm_num_n_tiles(N)
        tg = targets.to(torch.int32).contiguous()
        pm = torch.empty((3, parts, M), dtype=torch.float32, device=dev)
        tl = torch.zeros(M, dtype=torch.float32, device=dev)
        logp = torch.empty(M, dtype=torch.float32, device=dev)
        ent = torch.empty(M, dtype=torch.float32, device=dev)
        lse = torch.empty(M, dtype=torch.float32, device=dev)
        call("rlb_lm_head_logprob", ptr(h), ptr(w), M, N, K, h.stride(0), w.stride(0), ptr(tg), inv_temp,
             ptr(pm[0]), ptr(pm[1]), ptr(pm[2]), ptr(tl), ptr(logp), ptr(ent), ptr(lse),
             ptr(_L.status_word(dev)), stream_ptr())
        ctx.save_for_backward(h, w, tg, lse, ent)
        ctx.inv_temp = inv_temp
        ctx.want_entropy = want_entropy
        return logp, (ent if want_entropy else None)

    @staticmethod
    def backward(ctx, dlogp, dent):
        h, w, tg, lse, ent = ctx.saved_tensors
        M, K = h.shape
        N = w.shape[0]
        dev = h.device
        coef = dlogp.float().contiguous()
        ecoef = dent.float().contiguous() if (dent is not None and ctx.want_entropy) else None
        dh = torch.empty_like(h) if ctx.needs_input_grad[0] else None
        main_grad = getattr(w, "main_grad", None)
        dw = None
        if ctx.needs_input_grad[1] and main_grad is None:
            dw = torch.zeros((N, K), dtype=torch.float32, device=dev)
        wgrad_target = main_grad if main_grad is not None else dw
        chunk = _LMHeadLogprob.CHUNK
        dz = torch.empty((min(chunk, M), N), dtype=BF16, device=dev)
        for s in range(0, M, chunk):
            e = min(M, s + chunk)
            m = e - s
            dzc = dz[:m]
            call("rlb_lm_head_dlogits", ptr(h[s:e]), ptr(w), ptr(dzc), m, N, K, h.stride(0), w.stride(0), dzc.stride(0),
                 ptr(tg[s:e]), ctx.inv_temp, ptr(lse[s:e]), ptr(coef[s:e]), ptr(ecoef[s:e]) if ecoef is not None else None,
                 ptr(ent[s:e]), ptr(_L.status_word(dev)), stream_ptr())
            if dh is not None:
                gemm(dzc, w, b_mn=True, out=dh[s:e])
            if wgrad_target is not None:
                gemm(dzc, h[s:e], a_mn=True, b_mn=True, out=wgrad_target, accumulate=True)
        if dw is not None:
            dw = dw.to(w.dtype)
        return dh, dw, None, None, None


def lm_head_logprobs(h: torch.Tensor, w: torch.Tensor, targets: torch.Tensor, temperature: float = 1.0,
                     want_entropy: bool = False):
    """Per-token log-probability of ``targets`` (and optionally the entropy) under softmax(h @ w^T / temperature).

    ``h`` [T, d], ``w`` [V, d], ``targets`` [T]. fp32 results. The native path fuses the projection with the
    softmax statistics (the [T, V] logits are never stored), the role that
    ``ChunkedDistributedHiddenStatesToLogprobs`` plays in the reference (nemo_rl/distributed/model_utils.py:2137-2316).
    """
    inv_temp = 1.0 / temperature
    if not use_native(h):
        return _lm_head_ref(h, w, targets, inv_temp, want_entropy)
    h = h if h.stride(-1) == 1 else h.contiguous()
    return _LMHeadLogprob.apply(h, w, targets, inv_temp, want_entropy)


# --------------------------------------------------------------------------------------- optimizer pieces
def adamw_step(p_bf16, p_lo, p32, grad, m, v, *, lr, beta1, beta2, eps, weight_decay, step, grad_scale=None):
    """One AdamW update over a flat shard. Master weight is ``p32`` (fp32) or the split pair (``p_bf16``, ``p_lo``)."""
    n = m.numel()
    if not use_native(m):
        w = p32.clone() if p32 is not None else join_master(p_bf16, p_lo)
        g = grad.float() * (grad_scale.item() if grad_scale is not None else 1.0)
        m.mul_(beta1).add_(g, alpha=1 - beta1)
        v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
        w = w * (1 - lr * weight_decay)
        w = w - lr * (m / (1 - beta1**step)) / ((v / (1 - beta2**step)).sqrt() + eps)
        if p32 is not None:
            p32.copy_(w)
            if p_bf16 is not None:
                p_bf16.copy_(w.to(BF16))
        else:
            hi, lo = split_master(w)
            p_bf16.copy_(hi)
            p_lo.copy_(lo)
        return
    call("rlb_adamw", ptr(p_bf16), ptr(p_lo), ptr(p32), ptr(grad), int(grad.dtype == BF16), ptr(m), ptr(v), n,
         lr, beta1, beta2, eps, weight_decay, step, ptr(grad_scale), stream_ptr())


def split_master(w32: torch.Tensor):
    """fp32 -> (bf16, int16 remainder) with ``bits(w32) == (bits(hi) << 16) + lo`` exactly.

    The bf16 half rounds to nearest with ties away from zero, so the remainder always fits 16 signed bits."""
    bits = w32.contiguous().view(torch.int32)
    hb = (bits + 0x8000) & -65536
    hi = (hb >> 16).to(torch.int16).view(BF16)
    lo = (bits - hb).to(torch.int16)
    return hi, lo


def join_master(hi: torch.Tensor, lo: torch.Tensor) -> torch.Tensor:
    bits = (hi.view(torch.int16).to(torch.int32) << 16) + lo.to(torch.int32)
    return bits.view(torch.float32)


def sumsq_(x: torch.Tensor, out: torch.Tensor) -> None:
    """out += sum(x^2) (out: 1-element fp32 tensor on the same device)."""
    if not use_native(x):
        out.add_(x.float().pow(2).sum())
        return
    call("rlb_sumsq", ptr(x), int(x.dtype == BF16), x.numel(), ptr(out), stream_ptr())


def clip_scale(sumsq: torch.Tensor, max_norm: float, extra: float, scale_out: torch.Tensor, norm_out: torch.Tensor) -> None:
    if not use_native(sumsq):
        norm = sumsq.sqrt()
        norm_out.copy_(norm)
        s = torch.clamp(max_norm / (norm + 1e-6), max=1.0) if max_norm > 0 else torch.ones_like(norm)
        scale_out.copy_(s * extra)
        return
    call("rlb_clip_scale", ptr(sumsq), float(max_norm), float(extra), ptr(scale_out), ptr(norm_out), stream_ptr())
