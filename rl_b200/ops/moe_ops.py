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
    ``down`` [E, d, f]. Returns the experts' outputs [n, d] in the order of ``xs``. Parameters that carry quantisation-aware
    training quantizers (``rl_b200/policy/qat.py``) have them applied to their weights and to the rows entering them."""
    n, d = xs.shape
    E = gate_up.shape[0]
    if n == 0:
        return xs.new_zeros((0, d))
    q_up, q_down = getattr(gate_up, "_rlb_qat", None), getattr(down, "_rlb_qat", None)
    if q_up is not None or q_down is not None:
        from rl_b200.policy.qat import QatState

        if not QatState.enabled:
            q_up = q_down = None
    if q_up is not None:
        xs, gate_up = q_up.q_input(xs), q_up.q_weight(gate_up)
    if q_down is not None:
        down = q_down.q_weight(down)
    native = use_native(xs) and xs.dtype == BF16 and d % 64 == 0 and down.shape[2] % 64 == 0
    if not native:
        outs, s = [], 0
        for e, c in enumerate(counts.tolist()):
            if c:
                xe = xs[s : s + c]
                a = F.swiglu(F.linear(xe, gate_up[e]))
                outs.append(F.linear(a if q_down is None else q_down.q_input(a), down[e]))
                s += c
        return torch.cat(outs, 0) if outs else xs.new_zeros((0, d))
    lay = ExpertLayout(counts, n)
    xp = torch.zeros((lay.mpad, d), dtype=xs.dtype, device=xs.device).index_copy(0, lay.dest, xs)
    h = grouped_linear(xp, gate_up, lay)
    a = F.swiglu(h)
    if q_down is not None:
        a = q_down.q_input(a)
    y = grouped_linear(a, down, lay)
    return y.index_select(0, lay.dest)


# ------------------------------------------------------------------------------------------- small-token path (decode)
register("rlb_moe_route_topk", [P, L, I, I, I, I, P, P, P])
register("rlb_moe_decode_plan", [P, I, I, I, I, I, P, P, P, P, P, P, P])
register("rlb_moe_gather_rows", [P, L, P, P, P, I, I, P])
register("rlb_moe_combine", [P, P, P, P, P, I, I, I, P])

SMALL_MAX_COPIES = 16384   # token copies (tokens x top-k, all ranks) the one-CTA layout kernel handles
SMALL_WORKSPACES: dict = {}  # single-rank workspaces by (device, hidden, inter, experts, top-k)


def route_topk_ref(logits: torch.Tensor, k: int, renorm: bool):
    probs = torch.softmax(logits.float(), dim=-1)
    w, idx = torch.topk(probs, k, dim=-1)
    return (w / w.sum(-1, keepdim=True) if renorm else w), idx.to(torch.int32)


def route_topk(logits: torch.Tensor, k: int, renorm: bool, out_w=None, out_idx=None):
    """Soft-max over the router logits [T, E] (bf16), the k largest probabilities and their experts (one kernel)."""
    if not (use_native(logits) and logits.dtype == BF16 and logits.stride(-1) == 1):
        return route_topk_ref(logits, k, renorm)
    T, E = logits.shape
    w = out_w if out_w is not None else torch.empty((T, k), dtype=torch.float32, device=logits.device)
    idx = out_idx if out_idx is not None else torch.empty((T, k), dtype=torch.int32, device=logits.device)
    call("rlb_moe_route_topk", ptr(logits), logits.stride(0), T, E, k, int(renorm), ptr(w), ptr(idx), stream_ptr())
    return w, idx


class SmallTokenMoE:
    """Buffers and launchers of the few-token MoE layer (rl_b200/csrc/moe_decode.cu): gather the tokens of all expert-
    parallel ranks, route them identically everywhere, run the local experts' grouped MLP over the copies routed to them
    and reduce the partial sums to the tokens' owners. Nine launches per layer, fixed shapes, no host visit: a decode
    step that contains it can be captured in a CUDA graph. One instance serves all layers of a model.

    With ``ep.world > 1`` every rank of the group must call :meth:`forward` with the same number of tokens (the generation
    engine pads its decode batches to a bucket the ranks agree on)."""

    def __init__(self, hidden: int, inter: int, num_experts: int, top_k: int, ep, max_tokens: int, device, wait_limit_s: float = 20.0):
        self.d, self.f, self.E, self.k = hidden, inter, num_experts, top_k
        self.ep = ep
        self.W = ep.world if ep is not None else 1
        self.rank = ep.rank if ep is not None else 0
        self.El = num_experts // self.W
        self.e_lo = self.rank * self.El
        self.maxT = int(max_tokens)
        self.device = device
        self.wait_limit_s = wait_limit_s
        n_all = self.W * self.maxT
        assert n_all * top_k <= SMALL_MAX_COPIES and hidden % 8 == 0 and self.El <= 256 and top_k <= 16
        self.max_mpad = self.mpad_for(self.maxT)
        i32 = dict(dtype=torch.int32, device=device)
        self.w = torch.empty((n_all, top_k), dtype=torch.float32, device=device)
        self.idx = torch.empty((n_all, top_k), **i32)
        self.src_tok = torch.empty(self.max_mpad, **i32)
        self.copy_row = torch.empty(n_all * top_k, **i32)
        self.tile_expert = torch.empty(self.max_mpad // 128, **i32)
        self.row0 = torch.empty(self.El, **i32)
        self.rows = torch.empty(self.El, **i32)
        self.xp = torch.empty((self.max_mpad, hidden), dtype=BF16, device=device)
        self.h = torch.empty((self.max_mpad, 2 * inter), dtype=BF16, device=device)
        self.y = torch.empty((self.max_mpad, hidden), dtype=BF16, device=device)
        self._sym = []
        if self.W > 1:
            import ctypes as C

            from rl_b200.parallel.symmetric import SymmetricBuffer

            lib = _L.lib()
            Pp, Ii, LL, D = C.c_void_p, C.c_int, C.c_longlong, C.c_double
            lib.rlb_p2p_gather_cols.argtypes = [Pp, Pp, Pp, Pp, LL, Ii, Ii, Ii, Ii, Pp, D, Pp, Pp, LL, Pp]
            lib.rlb_p2p_gather_cols.restype = C.c_int
            lib.rlb_moe_combine_reduce.argtypes = [Pp, Pp, Pp, Pp, Pp, Ii, Ii, Ii, Pp, Pp, Ii, Ii, Pp, D, Pp, Pp, LL, Pp]
            lib.rlb_moe_combine_reduce.restype = C.c_int
            self._lib = lib
            self.stage_x = SymmetricBuffer(2 * self.maxT * hidden * 2, ep.group)
            self.stage_y = SymmetricBuffer(2 * n_all * hidden * 4, ep.group)
            self.flags = SymmetricBuffer(256, ep.group)          # words 0..7: gather, words 32..39: reduce
            self._sym = [self.stage_x, self.stage_y, self.flags]
            self._flags_g = (C.c_void_p * self.W)(*self.flags.peer_ptrs)
            self._flags_r = (C.c_void_p * self.W)(*[p + 128 for p in self.flags.peer_ptrs])
            self.epochs = torch.zeros(2, dtype=torch.int32, device=device)
            self.scratch = torch.zeros(2, dtype=torch.int32, device=device)
            self.x_all = torch.empty((n_all, hidden), dtype=BF16, device=device)

    def mpad_for(self, T: int) -> int:
        return -(-(self.W * T * self.k + self.El * 127) // 128) * 128

    def fits(self, T: int) -> bool:
        return 0 < T <= self.maxT

    def forward(self, x: torch.Tensor, residual, router: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor, renorm: bool):
        """x [T, d] bf16 -> (residual +) MoE(x) [T, d]; also returns the top-k experts of this rank's tokens."""
        T, d = x.shape
        W, k = self.W, self.k
        n_all = W * T
        st = stream_ptr()
        status = ptr(_L.status_word(x.device))
        x = x if x.stride(1) == 1 and x.stride(0) == d else x.contiguous()
        if W > 1:
            xa = self.x_all[:n_all]
            rc = self._lib.rlb_p2p_gather_cols(x.data_ptr(), self.stage_x.table, self._flags_g, xa.data_ptr(), n_all * d * 2, 1, T * d * 2,
                                               self.rank, W, self.epochs[0:1].data_ptr(), float(self.wait_limit_s),
                                               self.scratch[0:1].data_ptr(), status, self.maxT * d * 2, st)
            _L.Counters.launches += 1
            if rc:
                raise RuntimeError(f"rlb_p2p_gather_cols failed with code {rc}")
        else:
            xa = x
        logits = F.linear(xa, router)
        wts, idx = self.w[:n_all], self.idx[:n_all]
        call("rlb_moe_route_topk", ptr(logits), logits.stride(0), n_all, self.E, k, int(renorm), ptr(wts), ptr(idx), st)
        mpad = self.mpad_for(T)
        call("rlb_moe_decode_plan", ptr(idx), n_all * k, k, self.e_lo, self.El, mpad, ptr(self.src_tok), ptr(self.copy_row),
             ptr(self.tile_expert), ptr(self.row0), ptr(self.rows), status, st)
        xp, h, y = self.xp[:mpad], self.h[:mpad], self.y[:mpad]
        call("rlb_moe_gather_rows", ptr(xa), xa.stride(0) * 2, ptr(self.src_tok), ptr(self.tile_expert), ptr(xp), mpad, d * 2, st)
        call("rlb_gemm_grouped_rows", ptr(xp), xp.stride(0), ptr(gate_up), 0, ptr(h), h.stride(0), mpad, 2 * self.f, d, self.El,
             ptr(self.tile_expert), 0, status, st)
        a = F.swiglu(h)
        call("rlb_gemm_grouped_rows", ptr(a), a.stride(0), ptr(down), 0, ptr(y), y.stride(0), mpad, d, self.f, self.El,
             ptr(self.tile_expert), 0, status, st)
        out = torch.empty((T, d), dtype=BF16, device=x.device)
        res = ptr(residual.contiguous()) if residual is not None else None
        if W > 1:
            rc = self._lib.rlb_moe_combine_reduce(y.data_ptr(), self.copy_row.data_ptr(), wts.data_ptr(), res, out.data_ptr(), T, k, d,
                                                  self.stage_y.table, self._flags_r, self.rank, W, self.epochs[1:2].data_ptr(),
                                                  float(self.wait_limit_s), self.scratch[1:2].data_ptr(), status, W * self.maxT * d * 4, st)
            _L.Counters.launches += 1
            if rc:
                raise RuntimeError(f"rlb_moe_combine_reduce failed with code {rc}")
            mine = idx[self.rank * T : (self.rank + 1) * T]
        else:
            call("rlb_moe_combine", ptr(y), ptr(self.copy_row), ptr(wts), res, ptr(out), T, k, d, st)
            mine = idx
        return out, mine

    def close(self) -> None:
        for b in self._sym:
            b.close()
        self._sym = []
