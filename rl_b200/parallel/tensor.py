"""Tensor parallelism with sequence parallelism: column / row parallel linears whose collectives are fused into the
GEMM kernels on NVLink-connected GPUs (rl_b200/csrc/gemm_tp.cu), with ``torch.distributed`` twins (NCCL on GPUs without
the fused path, gloo on CPU).

Layouts (``tp`` ranks, packed token stream of ``T`` rows, ``T % tp == 0``):
  * between blocks activations are *sequence parallel*: rank r holds rows [r*T/tp, (r+1)*T/tp)
  * ``gather_linear(x_local, W_col)``   all-gather rows -> Y[T, N/tp] = X W_col^T             (qkv, gate_up)
  * ``linear_scatter(a, W_row, res)``   Y_partial[T, d] = A W_row^T -> reduce-scatter rows (+ residual)  (o, down)
  * ``linear_allreduce(a, W_row, res)`` the same with an all-reduce: every rank keeps all rows (decode, tp without sp)
Backward passes are the mirror images (all-gather <-> reduce-scatter), so every collective of a layer rides inside a GEMM
kernel. The reference gets these semantics from DTensor ``ColwiseParallel`` / ``RowwiseParallel`` /
``SequenceParallel`` plans (nemo_rl/models/dtensor/parallelize.py:355-470) or Megatron's tensor-parallel layers.
"""

from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
import torch.distributed as dist

from rl_b200.ops import functional as F
from rl_b200.ops import lib as _L
from rl_b200.ops.lib import use_native

BF16 = torch.bfloat16


# --------------------------------------------------------------------------------------------- twins (NCCL / gloo)
def all_gather_rows(x: torch.Tensor, group, world: int) -> torch.Tensor:
    if world == 1:
        return x
    x = x.contiguous()
    out = torch.empty((world * x.shape[0], *x.shape[1:]), dtype=x.dtype, device=x.device)
    if x.is_cuda:
        dist.all_gather_into_tensor(out, x, group=group)
    else:
        dist.all_gather(list(out.chunk(world, 0)), x, group=group)
    return out


def reduce_scatter_rows(y: torch.Tensor, group, world: int, rank: int) -> torch.Tensor:
    if world == 1:
        return y
    y = y.contiguous()
    rows = y.shape[0] // world
    if y.is_cuda:
        out = torch.empty((rows, *y.shape[1:]), dtype=y.dtype, device=y.device)
        dist.reduce_scatter_tensor(out, y, op=dist.ReduceOp.SUM, group=group)
        return out
    dist.all_reduce(y, op=dist.ReduceOp.SUM, group=group)  # gloo has no reduce-scatter
    return y[rank * rows : (rank + 1) * rows].clone()


def all_reduce_(y: torch.Tensor, group, world: int) -> torch.Tensor:
    if world > 1:
        dist.all_reduce(y, op=dist.ReduceOp.SUM, group=group)
    return y


# --------------------------------------------------------------------------------------------- fused peer-memory path
_P, _I, _LL, _D, _U = C.c_void_p, C.c_int, C.c_longlong, C.c_double, C.c_uint
_bound = False


def _bind():
    global _bound
    lib = _L.lib()
    if not _bound:
        lib.rlb_gemm_tp_gather.argtypes = [_P, _LL, _P, _LL, _I, _P, _LL, _P, _I, _I, _I, _P, _P, _I, _I, _U, _I, _D, _P, _P]
        lib.rlb_gemm_tp_scatter.argtypes = [_P, _LL, _P, _LL, _I, _I, _I, _I, _I, _I, _P, _LL, _P, _LL, _P, _P, _I, _I, _U, _P, _D, _P, _P]
        lib.rlb_p2p_gather_cols.argtypes = [_P, _P, _P, _P, _LL, _I, _I, _I, _I, _P, _D, _P, _P, _LL, _P]
        lib.rlb_p2p_gather_cols.restype = C.c_int
        lib.rlb_p2p_allreduce_rows.argtypes = [_P, _P, _P, _P, _P, C.c_float, _I, _I, _P, _P, _I, _I, _P, _D, _P, _P, _LL, _P]
        lib.rlb_p2p_allreduce_rows.restype = C.c_int
        lib.rlb_gemm_tp_gather.restype = C.c_int
        lib.rlb_gemm_tp_scatter.restype = C.c_int
        _bound = True
    return lib


class TPFusedComm:
    """Symmetric staging buffers + flags of one tensor-parallel group, and launchers of the fused kernels.

    ``max_rows`` is the largest gathered row count (tokens of a micro-batch), ``max_cols`` the widest gathered /
    scattered matrix (the hidden size). Buffers grow on demand (collectively: all ranks see the same shapes)."""

    def __init__(self, group, max_rows: int = 0, max_cols: int = 0, wait_limit_s: float = 10.0, pushers: int = 12):
        from rl_b200.parallel.symmetric import SymmetricBuffer

        self._SB = SymmetricBuffer
        self.group = group
        self.wait_limit_s = wait_limit_s
        self.pushers = pushers
        self.ctrl = SymmetricBuffer(1024, group)  # gather flags at 0, scatter flags at 256, column-gather flags at 512
        self.rank, self.world = self.ctrl.rank, self.ctrl.world
        self._gflags = (_P * self.world)(*self.ctrl.peer_ptrs)
        self._sflags = (_P * self.world)(*[p + 256 for p in self.ctrl.peer_ptrs])
        self._cflags = (_P * self.world)(*[p + 512 for p in self.ctrl.peer_ptrs])
        self._rflag_buf = None      # per-row flag words of the one-shot all-reduce (allocated at first use)
        self._rflags = None
        self.stage_r = None
        self.epoch_r_dev = torch.zeros(1, dtype=torch.int32, device=self.ctrl.device)
        self._r_scratch = torch.zeros(1, dtype=torch.int32, device=self.ctrl.device)
        self.stage_l = None
        self.epoch_c_dev = torch.zeros(1, dtype=torch.int32, device=self.ctrl.device)
        self._c_scratch = torch.zeros(1, dtype=torch.int32, device=self.ctrl.device)
        self.stage_a = None
        self.stage_c = None
        self.epoch_g = 0
        # the scatter kernel keeps its epoch in device memory, so launches replayed from a CUDA graph stay in step
        self.epoch_s_dev = torch.zeros(1, dtype=torch.int32, device=self.ctrl.device)
        if max_rows and max_cols:
            self._ensure("stage_a", max_rows * max_cols * 2)
            self._ensure("stage_c", max_rows * max_cols * 2)

    def _ensure(self, name: str, nbytes: int):
        buf = getattr(self, name)
        if buf is None or buf.nbytes < nbytes:
            if buf is not None:
                buf.close()
            setattr(self, name, self._SB(int(nbytes * 1.25) if buf is not None else nbytes, self.group))
        return getattr(self, name)

    def gathered(self, rows_total: int, K: int) -> torch.Tensor:
        """The gathered A of the last ``gather_gemm`` call ([rows_total, K] view of the local staging buffer)."""
        return self.stage_a.tensor(BF16, rows_total * K).view(rows_total, K)

    def gather_gemm(self, x_local: torch.Tensor, w: torch.Tensor, b_mn: bool = False, bias: Optional[torch.Tensor] = None,
                    out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Y[world*rows, N] = allgather(x_local) @ (w^T if not b_mn else w)."""
        lib = _bind()
        rows, K = x_local.shape
        N = w.shape[1] if b_mn else w.shape[0]
        assert x_local.dtype == BF16 and w.dtype == BF16 and x_local.stride(1) == 1 and w.stride(1) == 1
        st = self._ensure("stage_a", self.world * rows * K * 2)
        if out is None:
            out = torch.empty((self.world * rows, N), dtype=BF16, device=x_local.device)
        self.epoch_g += 1
        bias32 = bias.float() if bias is not None and bias.dtype != torch.float32 else bias
        rc = lib.rlb_gemm_tp_gather(x_local.data_ptr(), x_local.stride(0), w.data_ptr(), w.stride(0), int(b_mn), out.data_ptr(),
                                    out.stride(0), None if bias32 is None else bias32.data_ptr(), rows, N, K, st.table, self._gflags,
                                    self.rank, self.world, self.epoch_g, self.pushers, float(self.wait_limit_s),
                                    _L.status_word(x_local.device).data_ptr(), torch.cuda.current_stream().cuda_stream)
        _L.Counters.launches += 1
        if rc:
            raise RuntimeError(f"rlb_gemm_tp_gather failed with code {rc}")
        return out

    def scatter_gemm(self, a: torch.Tensor, w: torch.Tensor, b_mn: bool = False, residual: Optional[torch.Tensor] = None,
                     all_reduce: bool = False) -> torch.Tensor:
        """reduce_scatter_rows(a @ op(w)) (+ residual), or the all-reduced full result when ``all_reduce``."""
        lib = _bind()
        M, K = a.shape
        N = w.shape[1] if b_mn else w.shape[0]
        assert a.dtype == BF16 and w.dtype == BF16 and a.stride(1) == 1 and w.stride(1) == 1
        rows = M if all_reduce else M // self.world
        st = self._ensure("stage_c", self.world * rows * N * 2)
        out = torch.empty((rows, N), dtype=BF16, device=a.device)
        if residual is not None:
            assert residual.shape == out.shape and residual.dtype == BF16 and residual.stride(1) == 1
        rc = lib.rlb_gemm_tp_scatter(a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), int(b_mn), M, N, K, rows, int(all_reduce),
                                     out.data_ptr(), out.stride(0), None if residual is None else residual.data_ptr(),
                                     0 if residual is None else residual.stride(0), st.table, self._sflags, self.rank, self.world,
                                     0, self.epoch_s_dev.data_ptr(), float(self.wait_limit_s), _L.status_word(a.device).data_ptr(),
                                     torch.cuda.current_stream().cuda_stream)
        _L.Counters.launches += 1
        if rc:
            raise RuntimeError(f"rlb_gemm_tp_scatter failed with code {rc}")
        return out

    def gather_cols(self, z_local: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """[rows, world * n] from every rank's [rows, n] column slice over peer memory (vocabulary-parallel logits at
        decode time). No NCCL call and a device-resident epoch: the launch can be recorded in a CUDA graph."""
        lib = _bind()
        rows, n = z_local.shape
        z_local = z_local.contiguous()
        row_bytes = n * z_local.element_size()
        assert row_bytes % 16 == 0, "column slices must be a multiple of 16 bytes wide"
        # sized for 256 rows at the first call: decode batches of every bucket then share one stage whose two halves sit
        # at fixed offsets (a captured graph keeps the stage's address, and calls of different sizes never overlap)
        st = self._ensure("stage_l", 2 * max(rows, 256) * row_bytes)
        half_bytes = (st.nbytes // 2) // 16 * 16
        if out is None:
            out = torch.empty((rows, self.world * n), dtype=z_local.dtype, device=z_local.device)
        rc = lib.rlb_p2p_gather_cols(z_local.data_ptr(), st.table, self._cflags, out.data_ptr(), out.stride(0) * out.element_size(),
                                     rows, row_bytes, self.rank, self.world, self.epoch_c_dev.data_ptr(), float(self.wait_limit_s),
                                     self._c_scratch.data_ptr(), _L.status_word(z_local.device).data_ptr(), half_bytes,
                                     torch.cuda.current_stream().cuda_stream)
        _L.Counters.launches += 1
        if rc:
            raise RuntimeError(f"rlb_p2p_gather_cols failed with code {rc}")
        return out

    def allreduce_rows(self, partial: torch.Tensor, residual: Optional[torch.Tensor] = None, norm_w: Optional[torch.Tensor] = None,
                       eps: float = 1e-6, max_rows: int = 256):
        """Decode-sized all-reduce over peer memory: ``out = bf16(sum over ranks of partial + residual)`` on every rank, plus
        ``out2 = rmsnorm(out) * norm_w`` when ``norm_w`` is given (the norm that follows a row-parallel projection).
        ``partial`` [M, N] fp32 (M <= ``max_rows``). One launch, device-resident epoch: capturable in a CUDA graph."""
        lib = _bind()
        M, N = partial.shape
        assert partial.dtype == torch.float32 and partial.is_contiguous() and N % 8 == 0 and M <= max_rows
        st = self._ensure("stage_r", 2 * max_rows * N * 4)
        half_bytes = (st.nbytes // 2) // 16 * 16
        if self._rflag_buf is None:
            lib.rlb_p2p_allreduce_flag_bytes.restype = C.c_int
            self._rflag_buf = self._SB(int(lib.rlb_p2p_allreduce_flag_bytes()), self.group)
            self._rflags = (_P * self.world)(*self._rflag_buf.peer_ptrs)
        out = torch.empty((M, N), dtype=BF16, device=partial.device)
        out2 = torch.empty((M, N), dtype=BF16, device=partial.device) if norm_w is not None else None
        if residual is not None and not residual.is_contiguous():
            residual = residual.contiguous()
        rc = lib.rlb_p2p_allreduce_rows(partial.data_ptr(), residual.data_ptr() if residual is not None else None, out.data_ptr(),
                                        norm_w.data_ptr() if norm_w is not None else None, out2.data_ptr() if out2 is not None else None,
                                        float(eps), M, N, st.table, self._rflags, self.rank, self.world, self.epoch_r_dev.data_ptr(),
                                        float(self.wait_limit_s), self._r_scratch.data_ptr(), _L.status_word(partial.device).data_ptr(),
                                        half_bytes, torch.cuda.current_stream().cuda_stream)
        _L.Counters.launches += 1
        if rc:
            raise RuntimeError(f"rlb_p2p_allreduce_rows failed with code {rc}")
        return out, out2

    @staticmethod
    def phase_times_us() -> list[float]:
        """Durations (us) of the phases of the last ``scatter_gemm`` launch on this GPU, measured by CTA 0:
        [own tiles, first grid sync, peer barrier + second grid sync, reduce]."""
        lib = _bind()
        buf = (C.c_ulonglong * 5)()
        lib.rlb_gemm_tp_phase_times.argtypes = [C.POINTER(C.c_ulonglong)]
        lib.rlb_gemm_tp_phase_times.restype = C.c_int
        rc = lib.rlb_gemm_tp_phase_times(buf)
        if rc:
            raise RuntimeError(f"rlb_gemm_tp_phase_times failed with code {rc}")
        return [(buf[i + 1] - buf[i]) / 1e3 for i in range(4)]

    def close(self):
        for b in (self.stage_a, self.stage_c, self.stage_l, self.stage_r, self._rflag_buf, self.ctrl):
            if b is not None:
                b.close()


# --------------------------------------------------------------------------------------------- autograd functions
class TP:
    """Handle of one tensor-parallel group passed to the layers (``world == 1`` makes every op a plain linear)."""

    def __init__(self, group=None, rank: int = 0, world: int = 1, comm: Optional[TPFusedComm] = None, sequence_parallel: bool = False):
        self.group, self.rank, self.world, self.comm, self.sequence_parallel = group, rank, world, comm, sequence_parallel

    @classmethod
    def from_state(cls, st=None) -> "TP":
        from rl_b200.parallel.state import get_state

        st = st or get_state()
        return cls(st.tp_group, st.tp_rank, st.tp, st.tp_comm, st.sequence_parallel)

    def fused(self, x: torch.Tensor) -> bool:
        return self.comm is not None and x.is_cuda and x.dtype == BF16 and use_native(x)


def _accum_dw(w, dy2, x2):
    """dW[N, K] += dy^T x, straight into the gradient buffer when the parameter has one."""
    main_grad = getattr(w, "main_grad", None)
    if main_grad is not None:
        F.gemm(dy2, x2, a_mn=True, b_mn=True, out=main_grad, accumulate=True)
        return None
    return F.gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=w.dtype)


class _GatherLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_local, w, bias, tp: TP):
        ctx.tp = tp
        ctx.save_for_backward(x_local, w)
        ctx.has_bias = bias is not None
        if tp.fused(x_local):
            return tp.comm.gather_gemm(x_local, w, bias=bias)
        return F.gemm(all_gather_rows(x_local, tp.group, tp.world), w, bias=bias, out_dtype=x_local.dtype)

    @staticmethod
    def backward(ctx, dy):
        x_local, w = ctx.saved_tensors
        tp = ctx.tp
        dy = dy if dy.stride(-1) == 1 else dy.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            if tp.fused(dy):
                dx = tp.comm.scatter_gemm(dy, w, b_mn=True)
            else:
                dx = reduce_scatter_rows(F.gemm(dy, w, b_mn=True, out_dtype=x_local.dtype), tp.group, tp.world, tp.rank)
        if ctx.needs_input_grad[1]:
            dw = _accum_dw(w, dy, all_gather_rows(x_local, tp.group, tp.world))
        if ctx.has_bias:
            db = dy.float().sum(0).to(w.dtype)
        return dx, dw, db, None


class _LinearScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, w, residual, tp: TP, all_reduce: bool):
        ctx.tp, ctx.all_reduce = tp, all_reduce
        ctx.save_for_backward(a, w)
        ctx.has_res = residual is not None
        if tp.fused(a):
            return tp.comm.scatter_gemm(a, w, residual=residual, all_reduce=all_reduce)
        y = F.gemm(a, w, out_dtype=a.dtype)
        y = all_reduce_(y, tp.group, tp.world) if all_reduce else reduce_scatter_rows(y, tp.group, tp.world, tp.rank)
        return y if residual is None else y + residual

    @staticmethod
    def backward(ctx, dy):
        a, w = ctx.saved_tensors
        tp = ctx.tp
        dy = dy if dy.stride(-1) == 1 else dy.contiguous()
        da = dw = None
        if ctx.all_reduce:
            dy_full = dy
            if ctx.needs_input_grad[0]:
                da = F.gemm(dy_full, w, b_mn=True, out_dtype=a.dtype)
        elif tp.fused(dy):
            da = tp.comm.gather_gemm(dy, w, b_mn=True)
            dy_full = tp.comm.gathered(dy.shape[0] * tp.world, dy.shape[1])
        else:
            dy_full = all_gather_rows(dy, tp.group, tp.world)
            if ctx.needs_input_grad[0]:
                da = F.gemm(dy_full, w, b_mn=True, out_dtype=a.dtype)
        if ctx.needs_input_grad[1]:
            dw = _accum_dw(w, dy_full, a)
        return da, dw, (dy if ctx.has_res else None), None, None


class _ColumnLinear(torch.autograd.Function):
    """Column-parallel linear on a replicated input (tp without sequence parallelism): backward all-reduces dx."""

    @staticmethod
    def forward(ctx, x, w, bias, tp: TP):
        ctx.tp = tp
        ctx.save_for_backward(x, w)
        ctx.has_bias = bias is not None
        return F.gemm(x, w, bias=bias, out_dtype=x.dtype)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        tp = ctx.tp
        dy = dy if dy.stride(-1) == 1 else dy.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            if tp.fused(dy):
                dx = tp.comm.scatter_gemm(dy, w, b_mn=True, all_reduce=True)
            else:
                dx = all_reduce_(F.gemm(dy, w, b_mn=True, out_dtype=x.dtype), tp.group, tp.world)
        if ctx.needs_input_grad[1]:
            dw = _accum_dw(w, dy, x)
        if ctx.has_bias:
            db = dy.float().sum(0).to(w.dtype)
        return dx, dw, db, None


def column_linear(x: torch.Tensor, w: torch.Tensor, bias, tp: TP) -> torch.Tensor:
    """x: sequence-parallel rows (``tp.sequence_parallel``) or replicated rows -> all rows, this rank's output columns."""
    if tp.world == 1:
        return F.linear(x, w, bias)
    if tp.sequence_parallel:
        return _GatherLinear.apply(x, w, bias, tp)
    return _ColumnLinear.apply(x, w, bias, tp)


def row_linear(a: torch.Tensor, w: torch.Tensor, residual, tp: TP) -> torch.Tensor:
    """a: all rows, this rank's input columns -> summed output (+ residual): sequence-parallel rows or all rows."""
    if tp.world == 1:
        return F.linear(a, w, None, residual)
    return _LinearScatter.apply(a, w, residual, tp, not tp.sequence_parallel)


class _ScatterRows(torch.autograd.Function):
    """Replicated rows -> this rank's row shard (forward: slice, backward: all-gather)."""

    @staticmethod
    def forward(ctx, x, tp: TP):
        ctx.tp = tp
        rows = x.shape[0] // tp.world
        return x[tp.rank * rows : (tp.rank + 1) * rows].contiguous()

    @staticmethod
    def backward(ctx, dy):
        return all_gather_rows(dy, ctx.tp.group, ctx.tp.world), None


class _GatherRows(torch.autograd.Function):
    """Row shard -> all rows on every rank (forward: all-gather, backward: slice of the upstream gradient, which is
    identical on all ranks when the consumer is replicated)."""

    @staticmethod
    def forward(ctx, x, tp: TP):
        ctx.tp = tp
        return all_gather_rows(x, tp.group, tp.world)

    @staticmethod
    def backward(ctx, dy):
        tp = ctx.tp
        rows = dy.shape[0] // tp.world
        return dy[tp.rank * rows : (tp.rank + 1) * rows].contiguous(), None


def scatter_rows(x, tp: TP):
    return x if tp.world == 1 else _ScatterRows.apply(x, tp)


def gather_rows(x, tp: TP):
    return x if tp.world == 1 else _GatherRows.apply(x, tp)


class _GatherCols(torch.autograd.Function):
    """Column shards -> all columns on every rank (vocabulary-parallel logits -> full logits)."""

    @staticmethod
    def forward(ctx, x, tp: TP):
        ctx.tp = tp
        parts = all_gather_rows(x.t().contiguous(), tp.group, tp.world)  # [tp * n_local, T]
        return parts.t().contiguous()

    @staticmethod
    def backward(ctx, dy):
        tp = ctx.tp
        n = dy.shape[1] // tp.world
        return dy[:, tp.rank * n : (tp.rank + 1) * n].contiguous(), None


def gather_cols(x, tp: TP):
    return x if tp.world == 1 else _GatherCols.apply(x, tp)
