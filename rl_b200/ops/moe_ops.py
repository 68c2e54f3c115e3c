"""Mixture-of-experts compute: padded-by-expert token layout + grouped GEMMs (rl_b200/csrc/gemm_grouped.cu).

``grouped_expert_mlp(xs, counts, gate_up, down)`` runs the SwiGLU MLP of every local expert over its slice of ``xs``
(tokens sorted by expert, ``counts[e]`` rows each) with three launches in forward (two grouped GEMMs + SwiGLU) and no host
synchronisation: the per-expert segments are re-laid out with zero padding to multiples of 128 rows, so each 128-row tile
of the grouped GEMM belongs to one expert, and the tile -> expert table is computed on the device from ``counts``.
Weight gradients use the reduction form of the grouped GEMM and accumulate straight into the stacked gradient buffers.
On CPU (and for dtypes other than bf16) the per-expert loop of plain linears is used.
"""

from __future__ import annotations

import torch

from rl_b200.ops import functional as F
from rl_b200.ops import lib as _L
from rl_b200.ops.lib import I, L, P, call, ptr, register, stream_ptr, use_native

BF16 = torch.bfloat16
register("rlb_gemm_grouped_rows", [P, L, P, I, P, L, I, I, I, I, P, I, P, P])
register("rlb_gemm_grouped_reduce", [P, L, P, L, P, I, I, I, I, P, P, I, I, P, P])


class ExpertLayout:
    """Padded-by-expert row layout derived (on the device) from the per-expert row counts."""

    def __init__(self, counts: torch.Tensor, n_rows: int):
        E = counts.numel()
        dev = counts.device
        counts = counts.to(torch.int64)
        self.n_rows = n_rows
        self.num_experts = E
        self.mpad = -(-(n_rows + E * 127) // 128) * 128          # static upper bound: no host sync
        padded = (counts + 127) // 128 * 128
        ends = torch.cumsum(padded, 0)
        self.row0 = (ends - padded).to(torch.int32)
        self.rows = padded.to(torch.int32)
        start = torch.cumsum(counts, 0) - counts
        e_of_row = torch.repeat_interleave(torch.arange(E, device=dev), counts, output_size=n_rows)
        self.dest = (self.row0.long()[e_of_row] + torch.arange(n_rows, device=dev) - start[e_of_row])  # [n_rows] int64
        tile_start = torch.arange(self.mpad // 128, device=dev) * 128
        te = torch.searchsorted(ends, tile_start, right=True)
        self.tile_expert = torch.where(tile_start < ends[-1], te, torch.full_like(te, -1)).to(torch.int32)


class _GroupedLinear(torch.autograd.Function):
    """Y[Mpad, N] = X[Mpad, K] @ W[e(row)]^T with W stacked [E, N, K]."""

    @staticmethod
    def forward(ctx, x, w, lay: ExpertLayout):
        E, N, K = w.shape
        y = torch.zeros((lay.mpad, N), dtype=BF16, device=x.device)
        call("rlb_gemm_grouped_rows", ptr(x), x.stride(0), ptr(w), 0, ptr(y), y.stride(0), lay.mpad, N, K, E, ptr(lay.tile_expert), 0,
             ptr(_L.status_word(x.device)), stream_ptr())
        ctx.save_for_backward(x, w)
        ctx.lay = lay
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        lay = ctx.lay
        E, N, K = w.shape
        dy = dy if (dy.stride(-1) == 1 and dy.dtype == BF16) else dy.contiguous().to(BF16)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = torch.zeros((lay.mpad, K), dtype=BF16, device=dy.device)
            call("rlb_gemm_grouped_rows", ptr(dy), dy.stride(0), ptr(w), 1, ptr(dx), dx.stride(0), lay.mpad, K, N, E, ptr(lay.tile_expert),
                 0, ptr(_L.status_word(dy.device)), stream_ptr())
        if ctx.needs_input_grad[1]:
            main_grad = getattr(w, "main_grad", None)
            target = main_grad if main_grad is not None else torch.zeros((E, N, K), dtype=torch.float32, device=dy.device)
            call("rlb_gemm_grouped_reduce", ptr(dy), dy.stride(0), ptr(x), x.stride(0), ptr(target), lay.mpad, N, K, E, ptr(lay.row0),
                 ptr(lay.rows), int(target.dtype == torch.float32), 1, ptr(_L.status_word(dy.device)), stream_ptr())
            dw = None if main_grad is not None else target.to(w.dtype)
        return dx, dw, None


def grouped_linear(x_padded: torch.Tensor, w: torch.Tensor, lay: ExpertLayout) -> torch.Tensor:
    return _GroupedLinear.apply(x_padded, w, lay)


def grouped_expert_mlp(xs: torch.Tensor, counts: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    """``xs`` [n, d] sorted by (local) expert, ``counts`` [E] rows per expert (device tensor), ``gate_up`` [E, 2f, d],
    ``down`` [E, d, f]. Returns the experts' outputs [n, d] in the order of ``xs``."""
    n, d = xs.shape
    E = gate_up.shape[0]
    if n == 0:
        return xs.new_zeros((0, d))
    native = use_native(xs) and xs.dtype == BF16 and d % 64 == 0 and down.shape[2] % 64 == 0
    if not native:
        outs, s = [], 0
        for e, c in enumerate(counts.tolist()):
            if c:
                xe = xs[s : s + c]
                outs.append(F.linear(F.swiglu(F.linear(xe, gate_up[e])), down[e]))
                s += c
        return torch.cat(outs, 0) if outs else xs.new_zeros((0, d))
    lay = ExpertLayout(counts, n)
    xp = torch.zeros((lay.mpad, d), dtype=xs.dtype, device=xs.device).index_copy(0, lay.dest, xs)
    h = grouped_linear(xp, gate_up, lay)
    a = F.swiglu(h)
    y = grouped_linear(a, down, lay)
    return y.index_select(0, lay.dest)
