"""Weight synchronizer: executes a :class:`RefitPlan` with one copy kernel per rank (rl_b200/csrc/refit.cu).

Every rank owns a *weight arena* for its engine shard in peer-mapped memory. ``sync_weights()`` pushes the pieces of
this rank's trainer parameters that some engine rank needs straight into that rank's arena (local stores or P2P stores
over NVLink), then all ranks meet at a barrier; after it every arena holds the current weights in the engine's layout.
When trainer and engine share a layout no synchronizer is needed at all: the engine reads the trainer's buffers.

``WeightSynchronizer.twin_sync()`` is the collective form (all-gather of every HF tensor + slicing), the NCCL / gloo
baseline and the CPU path.
"""

from __future__ import annotations

import ctypes as C
import struct
from typing import Optional

import torch
import torch.distributed as dist

from rl_b200.models.config import ModelConfig
from rl_b200.models.transformer import CausalLM
from rl_b200.parallel.tensor import TP
from rl_b200.refit.plan import RefitPlan, build_refit_plan, serving_param_layout

WORK_VECS = 8192  # 128 KB per work item


def build_serving_model(cfg: ModelConfig, tp_serve: int, rank: int, arena: torch.Tensor, group=None, comm=None) -> CausalLM:
    """An engine-side model whose parameters are views into ``arena`` (laid out by :func:`serving_param_layout`)."""
    tp = TP(group, rank % tp_serve, tp_serve, comm, sequence_parallel=False)
    model = CausalLM(cfg, dtype=arena.dtype, device="meta", init=False, tp=tp)
    layout, total = serving_param_layout(cfg, tp_serve)
    assert arena.numel() >= total
    for name, p in list(model.named_parameters()):
        off, (r, c) = layout[name]
        view = arena[off : off + r * c].view(p.shape)
        mod = model
        *path, leaf = name.split(".")
        for part in path:
            mod = getattr(mod, part) if not part.isdigit() else mod[int(part)]
        setattr(mod, leaf, torch.nn.Parameter(view, requires_grad=False))
    from dataclasses import replace

    from rl_b200.models.config import rope_inv_freq

    model.inv_freq = rope_inv_freq(cfg, arena.device)
    if getattr(model, "inv_freq_local", None) is not None:
        model.inv_freq_local = rope_inv_freq(replace(cfg, rope_theta=cfg.rope_local_theta, rope_scaling=None), arena.device)
    for mod in model.modules():     # stored buffers (router selection biases): real storage, filled by the weight sync
        for bname, b in list(mod.named_buffers(recurse=False)):
            if b.is_meta:
                setattr(mod, bname, torch.zeros(b.shape, dtype=b.dtype, device=arena.device))
    return model


class WeightSynchronizer:
    def __init__(self, train_model: CausalLM, cfg: ModelConfig, tp_serve: int, group=None, serve_group=None, serve_comm=None):
        self.cfg = cfg
        self.train_model = train_model
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.group = group
        self.tp_train, self.tp_serve = train_model.tp.world, tp_serve
        self.plan: RefitPlan = build_refit_plan(cfg, self.world, self.tp_train, tp_serve)
        self.layout, self.arena_numel = serving_param_layout(cfg, tp_serve)
        p0 = next(train_model.parameters())
        self.dtype, self.device = p0.dtype, p0.device
        self.native = self.device.type == "cuda"
        self._sym = None
        if self.native and self.world > 1:
            from rl_b200.parallel.symmetric import SymmetricBuffer

            self._sym = SymmetricBuffer(self.arena_numel * p0.element_size(), group)
            self.arena = self._sym.tensor(self.dtype, self.arena_numel)
            self._arena_ptrs = list(self._sym.peer_ptrs)
        else:
            self.arena = torch.zeros(self.arena_numel, dtype=self.dtype, device=self.device)
            self._arena_ptrs = [self.arena.data_ptr()] * max(1, self.world)
        self.serving_model = build_serving_model(cfg, tp_serve, self.rank, self.arena, serve_group, serve_comm)
        self._descs = self._work = None
        self._token = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._num_work = 0
        self.last_bytes = 0

    # ------------------------------------------------------------------ native path
    def _prepare(self) -> None:
        from rl_b200.ops import lib as _L

        lib = _L.lib()
        params = dict(self.train_model.named_parameters())
        es = next(iter(params.values())).element_size()
        descs, work = [], []
        total = 0
        for op in self.plan.ops_from(self.rank):
            src = params[op.src_param].data_ptr() + op.src_offset * es
            dst = self._arena_ptrs[op.dst_rank] + (self.layout[op.dst_param][0] + op.dst_offset) * es
            row_bytes = op.row_elems * es
            # every copy is checked against the tensors it touches before anything reaches the device
            src_end = op.src_offset + (op.rows - 1) * op.src_pitch + op.row_elems
            dst_end = op.dst_offset + (op.rows - 1) * op.dst_pitch + op.row_elems
            d_off, (d_r, d_c) = self.layout[op.dst_param]
            if not (0 <= op.src_offset and src_end <= params[op.src_param].numel() and 0 <= op.dst_offset and dst_end <= d_r * d_c
                    and d_off + dst_end <= self.arena_numel and 0 <= op.dst_rank < max(1, self.world)):
                raise ValueError(f"refit op out of bounds: {op}")
            vec_ok = row_bytes % 16 == 0 and src % 16 == 0 and dst % 16 == 0 and (op.src_pitch * es) % 16 == 0 and (op.dst_pitch * es) % 16 == 0
            rows, sp, dp = op.rows, op.src_pitch * es, op.dst_pitch * es
            if rows > 1 and sp == row_bytes and dp == row_bytes:  # contiguous on both sides: one long row
                row_bytes, rows = row_bytes * rows, 1
            if row_bytes >= 2**31:
                split = -(-row_bytes // 2**30)
                assert rows == 1 and row_bytes % (16 * split) == 0
                parts = [(src + i * (row_bytes // split), dst + i * (row_bytes // split), row_bytes // split) for i in range(split)]
            else:
                parts = [(src, dst, row_bytes)]
            for s_, d_, rb in parts:
                di = len(descs)
                descs.append(struct.pack("<QQqqii", s_, d_, sp, dp, rows, rb))
                n = rows * (rb // 16) if vec_ok else rows * (rb // 2)
                for f in range(0, n, WORK_VECS):
                    work.append(struct.pack("<iiii", di, f, min(WORK_VECS, n - f), 0 if vec_ok else 1))
                total += rows * rb
        assert lib.rlb_refit_desc_bytes() == 40 and lib.rlb_refit_work_bytes() == 16
        self._descs = torch.frombuffer(bytearray(b"".join(descs) or b"\0" * 40), dtype=torch.uint8).to(self.device)
        self._work = torch.frombuffer(bytearray(b"".join(work) or b"\0" * 16), dtype=torch.uint8).to(self.device)
        self._num_work = len(work)
        self.last_bytes = total
        lib.rlb_refit_copy.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        lib.rlb_refit_copy.restype = C.c_int

    def sync_weights(self, timer=None) -> None:
        """Pushes this rank's pieces into every engine arena; returns after all ranks' pushes are complete."""
        if not self.native:
            return self.twin_sync()
        from rl_b200.ops import lib as _L

        if self._descs is None:
            self._prepare()
        # Stream-ordered rendezvous (a one-element all-reduce) instead of host barriers: the first makes sure no engine of
        # the group still reads its arena, the second that every peer's stores into this rank's arena have landed.
        if self.world > 1:
            dist.all_reduce(self._token, group=self.group)
        rc = _L.lib().rlb_refit_copy(self._descs.data_ptr(), self._work.data_ptr(), self._num_work, 0, torch.cuda.current_stream().cuda_stream)
        _L.Counters.launches += 1
        if rc:
            raise RuntimeError(f"rlb_refit_copy failed with code {rc}")
        if self.world > 1:
            dist.all_reduce(self._token, group=self.group)

    # ------------------------------------------------------------------ quantising push (FP8, 128 x 128 blocks)
    def _prepare_fp8(self) -> None:
        """Splits the plan: pieces of eligible linear weights made of whole 128 x 128 blocks go through the quantising
        kernel into an FP8 arena (e4m3 bytes + one fp32 de-scale per block, per serving parameter); everything else
        (norms, embeddings, the output head, ragged pieces) keeps the bf16 copy."""
        from rl_b200.engine.quantized import _eligible
        from rl_b200.ops import lib as _L

        lib = _L.lib()
        assert self.dtype == torch.bfloat16
        params = dict(self.train_model.named_parameters())
        serving = dict(self.serving_model.named_parameters())

        def blocks_ok(op) -> bool:
            _, (d_r, d_c) = self.layout[op.dst_param]
            r0, c0 = divmod(op.dst_offset, op.dst_pitch)
            return (op.dst_pitch == d_c and d_r % 128 == 0 and d_c % 128 == 0 and r0 % 128 == 0 and c0 % 128 == 0
                    and op.rows % 128 == 0 and op.row_elems % 128 == 0 and op.src_offset % 8 == 0 and op.src_pitch % 8 == 0)

        by_param: dict[str, list] = {}
        for op in self.plan.ops:
            by_param.setdefault(op.dst_param, []).append(op)
        fused = {n for n, ops in by_param.items() if n in serving and _eligible(n, serving[n], "fp8") and all(blocks_ok(o) for o in ops)}
        # FP8 arena layout (identical on every rank): per fused parameter its e4m3 bytes, then its de-scales
        off, q_layout = 0, {}
        for n in sorted(fused):
            _, (r, c) = self.layout[n]
            q_layout[n] = (off, off + r * c, r, c)
            off += r * c + (r // 128) * (c // 128) * 4
            off = -(-off // 256) * 256
        self._q_bytes = max(off, 256)
        if self.world > 1:
            from rl_b200.parallel.symmetric import SymmetricBuffer

            self._qsym = SymmetricBuffer(self._q_bytes, self.group)
            q_arena, q_ptrs = self._qsym.tensor(torch.uint8, self._q_bytes), list(self._qsym.peer_ptrs)
        else:
            self._qsym = None
            q_arena = torch.zeros(self._q_bytes, dtype=torch.uint8, device=self.device)
            q_ptrs = [q_arena.data_ptr()]
        self._q_arena = q_arena
        self._q_views = {}
        for n, (qo, so, r, c) in q_layout.items():
            q = q_arena[qo : qo + r * c].view(torch.float8_e4m3fn).view(r, c)
            sc = q_arena[so : so + (r // 128) * (c // 128) * 4].view(torch.float32).view(r // 128, c // 128)
            self._q_views[n] = (q, sc)
        # work lists
        qdescs, qwork, descs_rest = [], [], []
        es = 2
        self._q_remote = set()           # fused parameters with at least one block pushed by another rank: expanded after the barrier
        for op in self.plan.ops:
            if op.dst_param in fused and op.src_rank != op.dst_rank and op.dst_rank == self.rank:
                self._q_remote.add(op.dst_param)
        BLOCKS_PER_ITEM = 8
        total = 0
        for op in self.plan.ops_from(self.rank):
            if op.dst_param not in fused:
                descs_rest.append(op)
                continue
            qo, so, r, c = q_layout[op.dst_param]
            r0, c0 = divmod(op.dst_offset, op.dst_pitch)
            src = params[op.src_param].data_ptr() + op.src_offset * es
            dst_q = q_ptrs[op.dst_rank] + qo + op.dst_offset
            dst_s = q_ptrs[op.dst_rank] + so + ((r0 // 128) * (c // 128) + c0 // 128) * 4
            local = op.dst_rank == self.rank
            dst_w = (self._arena_ptrs[op.dst_rank] + (self.layout[op.dst_param][0] + op.dst_offset) * es) if local else 0
            src_end = op.src_offset + (op.rows - 1) * op.src_pitch + op.row_elems
            if not (0 <= op.src_offset and src_end <= params[op.src_param].numel() and r0 + op.rows <= r and c0 + op.row_elems <= c
                    and 0 <= op.dst_rank < max(1, self.world)):
                raise ValueError(f"refit op out of bounds: {op}")
            di = len(qdescs)
            bc = op.row_elems // 128
            qdescs.append(struct.pack("<QQQQqqii", src, dst_q, dst_s, dst_w, op.src_pitch, op.dst_pitch, c // 128, bc))
            nb = (op.rows // 128) * bc
            for f in range(0, nb, BLOCKS_PER_ITEM):
                qwork.append(struct.pack("<iiii", di, f, min(BLOCKS_PER_ITEM, nb - f), 0))
            total += op.rows * op.row_elems * es
        assert lib.rlb_refit_qdesc_bytes() == 56 and lib.rlb_refit_qwork_bytes() == 16
        self._qdescs = torch.frombuffer(bytearray(b"".join(qdescs) or b"\0" * 56), dtype=torch.uint8).to(self.device)
        self._qwork = torch.frombuffer(bytearray(b"".join(qwork) or b"\0" * 16), dtype=torch.uint8).to(self.device)
        self._num_qwork = len(qwork)
        self._fp8_fused = fused
        self._fp8_read_bytes = total
        # the bf16 copies that remain: a second plan restricted to the other parameters
        keep = self.plan
        self.plan = type(keep)(keep.world, keep.tp_train, keep.tp_serve, [o for o in keep.ops if o.dst_param not in fused])
        saved = (self._descs, self._work, self._num_work, self.last_bytes)
        self._descs = None
        self._prepare()
        self._rest = (self._descs, self._work, self._num_work)
        self._fp8_read_bytes += self.last_bytes
        self._descs, self._work, self._num_work, self.last_bytes = saved
        self.plan = keep
        lib.rlb_refit_quant.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        lib.rlb_refit_quant.restype = C.c_int

    def sync_weights_fp8(self) -> None:
        """Refit with block-128 FP8 weights for the engine in one pass over the trainer's weights: linear weights are
        quantised on the way (e4m3 + de-scales stored into the destination rank's FP8 arena; half the bytes of a bf16
        push cross NVLink), the other tensors are copied. Afterwards every eligible serving parameter carries its quantised
        form (``_rlb_q``) and the bf16 arena holds the fp8-rounded values the bf16 GEMMs compute with."""
        if not self.native:
            from rl_b200.engine.quantized import quantize_model

            self.twin_sync()
            quantize_model(self.serving_model, "fp8")
            return
        from rl_b200.ops import lib as _L
        from rl_b200.ops import quant as Q

        if getattr(self, "_qdescs", None) is None:
            self._prepare_fp8()
        lib = _L.lib()
        stream = torch.cuda.current_stream().cuda_stream
        if self.world > 1:
            dist.all_reduce(self._token, group=self.group)
        rd, rw, rn = self._rest
        rc = lib.rlb_refit_copy(rd.data_ptr(), rw.data_ptr(), rn, 0, stream) if rn else 0
        rc = rc or lib.rlb_refit_quant(self._qdescs.data_ptr(), self._qwork.data_ptr(), self._num_qwork, 0, stream)
        _L.Counters.launches += 2
        if rc:
            raise RuntimeError(f"quantising refit failed with code {rc}")
        if self.world > 1:
            dist.all_reduce(self._token, group=self.group)
        serving = dict(self.serving_model.named_parameters())
        for n in self._fp8_fused:
            q, sc = self._q_views[n]
            p = serving[n]
            if n in self._q_remote:      # blocks that arrived over NVLink as fp8: expand into the bf16 arena here
                Q.dequantize_fp8_blockwise_into(q, sc, p.data)
            p._rlb_q = ("fp8", q, sc)
            p._rlb_q_bf16 = p.data
        # eligible weights whose pieces were not whole blocks took the bf16 copy: quantise them in place
        from rl_b200.engine.quantized import _eligible

        for n, p in serving.items():
            if n not in self._fp8_fused and _eligible(n, p, "fp8"):
                q, sc = Q.quantize_fp8_blockwise(p.data)
                p._rlb_q = ("fp8", q, sc)
                p._rlb_q_bf16 = Q.dequantize_fp8_blockwise(q, sc)

    # ------------------------------------------------------------------ collective twin / CPU path
    @torch.no_grad()
    def twin_sync(self) -> None:
        from rl_b200.models.hf_io import iter_hf_tensors, load_hf_tensors

        full = {n: t.detach() for n, t in iter_hf_tensors(self.train_model)}
        load_hf_tensors(self.serving_model, full.get)

    def close(self) -> None:
        if getattr(self, "_qsym", None) is not None:
            self._qsym.close()
            self._qsym = None
        if self._sym is not None:
            self._sym.close()
