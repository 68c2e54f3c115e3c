"""Expert parallelism: token dispatch / combine between the ranks that share a MoE layer's experts.

Every rank routes its own tokens, sorts them by (global) expert, and sends each slice to the rank that owns the expert;
the owner runs its local experts over everything it received and sends the results back the same way. ``EP`` holds the
group; ``all_to_all_tokens`` is the differentiable dispatch -> experts -> combine round trip. The collective twin is
``torch.distributed.all_to_all_single`` (NCCL / gloo); on NVLink-connected GPUs the dispatch and combine copies go
through peer memory (rl_b200/csrc/moe_dispatch.cu) when an ``EPFusedComm`` is attached.

The reference delegates this step to Megatron's token dispatchers (allgather / alltoall / DeepEP flex,
nemo_rl/models/megatron/setup.py:888-1023; policy config ``moe_token_dispatcher_type``).
"""

from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist


class EP:
    def __init__(self, group=None, rank: int = 0, world: int = 1, comm=None):
        self.group, self.rank, self.world, self.comm = group, rank, world, comm

    @classmethod
    def from_state(cls, st=None) -> "EP":
        from rl_b200.parallel.state import get_state

        st = st or get_state()
        return cls(st.ep_group, st.ep_rank, st.ep, st.ep_comm)


class _AllToAllRows(torch.autograd.Function):
    """Rows of ``x`` are split by ``send`` (rows per destination) and received as ``recv`` (rows per source)."""

    @staticmethod
    def forward(ctx, x, send: list[int], recv: list[int], group):
        ctx.send, ctx.recv, ctx.group = send, recv, group
        out = torch.empty((sum(recv), *x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=recv, input_split_sizes=send, group=group)
        return out

    @staticmethod
    def backward(ctx, dy):
        dx = torch.empty((sum(ctx.send), *dy.shape[1:]), dtype=dy.dtype, device=dy.device)
        dist.all_to_all_single(dx, dy.contiguous(), output_split_sizes=ctx.send, input_split_sizes=ctx.recv, group=ctx.group)
        return dx, None, None, None


def exchange_counts(counts: torch.Tensor, ep: EP, local_experts: int) -> torch.Tensor:
    """``counts`` [E] tokens this rank sends to every global expert -> [ep, local_experts]: tokens each source rank sends
    to each of this rank's experts."""
    send = counts.view(ep.world, local_experts).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=ep.group)
    return recv


def all_to_all_tokens(xs: torch.Tensor, counts: torch.Tensor, ep: EP, local_experts: int,
                      expert_fn: Callable[[torch.Tensor, list[int]], torch.Tensor]) -> torch.Tensor:
    """``xs`` [n, d]: this rank's routed token copies sorted by global expert id, ``counts`` [E] their histogram.
    Returns the expert outputs in the same order as ``xs``."""
    recv_counts = exchange_counts(counts, ep, local_experts)            # [ep, local_experts]
    send_rows = counts.view(ep.world, local_experts).sum(1).tolist()
    rc = recv_counts.tolist()                                            # host sync: split sizes are data dependent
    recv_rows = [sum(r) for r in rc]
    got = _AllToAllRows.apply(xs, send_rows, recv_rows, ep.group)        # ordered by (source rank, local expert)
    # regroup by local expert so that each expert sees one contiguous slice
    n = got.shape[0]
    seg_start, off = [], 0
    for r in range(ep.world):
        for e in range(local_experts):
            seg_start.append((e, r, off, rc[r][e]))
            off += rc[r][e]
    order = []
    for e in range(local_experts):
        for (ee, r, o, c) in seg_start:
            if ee == e and c:
                order.append(torch.arange(o, o + c, device=xs.device))
    perm = torch.cat(order) if order else torch.empty(0, dtype=torch.long, device=xs.device)
    per_expert = [sum(rc[r][e] for r in range(ep.world)) for e in range(local_experts)]
    ys = expert_fn(got[perm] if n else got, per_expert)
    back = torch.empty_like(ys)
    if n:
        back[perm] = ys
    return _AllToAllRows.apply(back, recv_rows, send_rows, ep.group)


# --------------------------------------------------------------------------------------------- fused peer-memory path
class EPFusedComm:
    """Symmetric receive / return buffers of one expert-parallel group and launchers of the P2P dispatch kernels
    (rl_b200/csrc/moe_dispatch.cu). ``max_copies``: the largest number of routed token copies (tokens x top-k) one rank
    sends in one call; the receive buffer is sized for the worst case (every copy of every rank lands on one rank), so no
    token is ever dropped."""

    def __init__(self, group, hidden: int, max_copies: int, local_experts: int, dtype=torch.bfloat16, wait_limit_s: float = 10.0):
        import ctypes as C

        from rl_b200.ops import lib as _L
        from rl_b200.parallel.symmetric import SymmetricBuffer

        self.group = group
        self.hidden, self.local_experts, self.dtype = hidden, local_experts, dtype
        self.wait_limit_s = wait_limit_s
        self.ctrl = SymmetricBuffer(256, group)
        self.rank, self.world = self.ctrl.rank, self.ctrl.world
        self.max_copies = int(max_copies)
        self.cap_rows = -(-(self.world * self.max_copies + local_experts * 127) // 128) * 128
        es = torch.empty((), dtype=dtype).element_size()
        self.recv = SymmetricBuffer(self.cap_rows * hidden * es, group)
        self.meta = SymmetricBuffer(self.cap_rows * 8, group)
        self.ret = SymmetricBuffer(self.max_copies * hidden * es, group)
        self.epoch = [0, 0]
        lib = _L.lib()
        P, I, LL, U, D = C.c_void_p, C.c_int, C.c_longlong, C.c_uint, C.c_double
        lib.rlb_moe_push_rows.argtypes = [P, LL, P, P, P, I, I, P, P, P, I, I, I, U, D, P, LL, P]
        lib.rlb_moe_return_rows.argtypes = [P, LL, P, P, I, I, P, P, I, I, I, U, D, P, LL, P]
        lib.rlb_moe_push_rows.restype = lib.rlb_moe_return_rows.restype = C.c_int
        self._lib, self._L = lib, _L

    def recv_rows(self, rows: int) -> torch.Tensor:
        return self.recv.tensor(self.dtype, rows * self.hidden).view(rows, self.hidden)

    def ret_rows(self, rows: int) -> torch.Tensor:
        return self.ret.tensor(self.dtype, rows * self.hidden).view(rows, self.hidden)

    def meta_rows(self, rows: int) -> torch.Tensor:
        return self.meta.tensor(torch.int32, rows * 2).view(rows, 2)

    def push(self, src: torch.Tensor, dst_rank: torch.Tensor, dst_row: torch.Tensor, record_meta: bool) -> None:
        """Rows of ``src`` -> row ``dst_row[i]`` of rank ``dst_rank[i]``'s receive buffer; returns after every rank's push."""
        n, d = src.shape
        assert d == self.hidden and src.dtype == self.dtype and src.stride(1) == 1 and n <= self.max_copies
        self.epoch[0] += 1
        rc = self._lib.rlb_moe_push_rows(src.data_ptr(), src.stride(0) * src.element_size(), None, dst_rank.data_ptr(), dst_row.data_ptr(),
                                         n, d * src.element_size(), self.recv.table, self.meta.table if record_meta else None,
                                         self.ctrl.table, self.rank, self.world, 0, self.epoch[0], float(self.wait_limit_s),
                                         self._L.status_word(src.device).data_ptr(), self.cap_rows, torch.cuda.current_stream().cuda_stream)
        self._L.Counters.launches += 1
        if rc:
            raise RuntimeError(f"rlb_moe_push_rows failed with code {rc}")

    def give_back(self, src: torch.Tensor, meta: torch.Tensor, valid: torch.Tensor) -> None:
        """Row j of ``src`` -> rank ``meta[j, 0]``, row ``meta[j, 1]`` of that rank's return buffer (valid rows only)."""
        n, d = src.shape
        self.epoch[1] += 1
        rc = self._lib.rlb_moe_return_rows(src.data_ptr(), src.stride(0) * src.element_size(), meta.data_ptr(), valid.data_ptr(), n,
                                           d * src.element_size(), self.ret.table, self.ctrl.table, self.rank, self.world, 1,
                                           self.epoch[1], float(self.wait_limit_s), self._L.status_word(src.device).data_ptr(),
                                           self.max_copies, torch.cuda.current_stream().cuda_stream)
        self._L.Counters.launches += 1
        if rc:
            raise RuntimeError(f"rlb_moe_return_rows failed with code {rc}")

    def close(self):
        for b in (self.recv, self.meta, self.ret, self.ctrl):
            b.close()


class _DispatchPlan:
    """Where this rank's sorted token copies go, and how this rank's receive buffer is laid out (all on the device)."""

    def __init__(self, counts: torch.Tensor, ep: EP, local_experts: int, n: int):
        comm = ep.comm
        W, El = ep.world, local_experts
        dev = counts.device
        allc = torch.empty((W, W * El), dtype=torch.int64, device=dev)
        dist.all_gather_into_tensor(allc, counts.to(torch.int64).contiguous(), group=ep.group)
        per = allc.view(W, W, El)                       # [source, dest rank, local expert]
        total = per.sum(0)                              # [dest rank, local expert] rows received
        padded = (total + 127) // 128 * 128
        row0 = torch.cumsum(padded, 1) - padded         # [dest rank, local expert]
        before_me = per[: ep.rank].sum(0) if ep.rank > 0 else torch.zeros_like(total)
        my_off = (row0 + before_me).reshape(-1)         # [E] first row of my segment inside (rank, expert)
        c = counts.to(torch.int64)
        start = torch.cumsum(c, 0) - c
        e_of = torch.repeat_interleave(torch.arange(W * El, device=dev), c, output_size=n)
        self.n = n
        self.dst_rank = (e_of // El).to(torch.int32)
        self.dst_row = (my_off[e_of] + torch.arange(n, device=dev) - start[e_of]).to(torch.int32)
        # my own receive layout. The receive buffer is sized for the worst case (every copy of every rank lands here), but
        # everything downstream (masking, grouped GEMMs, SwiGLU, the return trip) only has to cover the rows that did
        # arrive: one small host read per call buys back passes over gigabytes of unused rows.
        mine_total, mine_pad, mine_row0 = total[ep.rank], padded[ep.rank], row0[ep.rank]
        need = int(mine_pad.sum().item())
        if need > comm.cap_rows:
            raise RuntimeError(f"expert-parallel receive buffer too small: {need} rows arrive, {comm.cap_rows} fit")
        self.mpad = max(128, need)
        self.row0 = mine_row0.to(torch.int32)
        self.rows = mine_pad.to(torch.int32)
        ends = torch.cumsum(mine_pad, 0)
        tile_start = torch.arange(self.mpad // 128, device=dev) * 128
        te = torch.searchsorted(ends, tile_start, right=True).clamp(max=El - 1)
        self.tile_expert = torch.where(tile_start < ends[-1], te, torch.full_like(te, -1)).to(torch.int32)
        r = torch.arange(self.mpad, device=dev)
        e_row = torch.searchsorted(ends, r, right=True).clamp(max=El - 1)
        self.valid = ((r < ends[-1]) & (r - mine_row0[e_row] < mine_total[e_row])).to(torch.int32)
        self.meta = None


class _P2PDispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, xs, plan: _DispatchPlan, comm: EPFusedComm):
        comm.push(xs.contiguous(), plan.dst_rank, plan.dst_row, record_meta=True)
        plan.meta = comm.meta_rows(plan.mpad).clone()
        ctx.plan, ctx.comm = plan, comm
        return comm.recv_rows(plan.mpad) * plan.valid.to(xs.dtype).unsqueeze(1)  # fresh tensor, padding rows zeroed

    @staticmethod
    def backward(ctx, d_recv):
        plan, comm = ctx.plan, ctx.comm
        comm.give_back(d_recv.contiguous(), plan.meta, plan.valid)
        return comm.ret_rows(plan.n).clone(), None, None


class _P2PCombine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y_rows, plan: _DispatchPlan, comm: EPFusedComm):
        comm.give_back(y_rows.contiguous(), plan.meta, plan.valid)
        ctx.plan, ctx.comm = plan, comm
        return comm.ret_rows(plan.n).clone()

    @staticmethod
    def backward(ctx, d_ret):
        plan, comm = ctx.plan, ctx.comm
        comm.push(d_ret.contiguous(), plan.dst_rank, plan.dst_row, record_meta=False)
        return comm.recv_rows(plan.mpad) * plan.valid.to(d_ret.dtype).unsqueeze(1), None, None


def fused_dispatch_experts_combine(xs: torch.Tensor, counts: torch.Tensor, ep: EP, local_experts: int, gate_up, down) -> torch.Tensor:
    """The peer-memory form of :func:`all_to_all_tokens` with the grouped-GEMM expert MLP in the middle."""
    from rl_b200.ops import functional as F
    from rl_b200.ops.moe_ops import ExpertLayout, grouped_linear

    plan = _DispatchPlan(counts, ep, local_experts, xs.shape[0])
    xp = _P2PDispatch.apply(xs, plan, ep.comm)
    lay = ExpertLayout.__new__(ExpertLayout)
    lay.n_rows, lay.num_experts, lay.mpad = xs.shape[0], local_experts, plan.mpad
    lay.row0, lay.rows, lay.tile_expert, lay.dest = plan.row0, plan.rows, plan.tile_expert, None
    y = grouped_linear(F.swiglu(grouped_linear(xp, gate_up, lay)), down, lay)
    return _P2PCombine.apply(y, plan, ep.comm)
