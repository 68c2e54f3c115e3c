"""Refit planning: which bytes of which trainer shard go where in which engine rank's weight arena.

Both sides are described by the same HuggingFace-name mapping (:func:`rl_b200.models.hf_io.hf_name_map`): a training
rank holds, for every HF tensor, a slice ``(dim, start, length)`` stored in some rows of a fused local parameter; a
serving rank needs another slice stored in rows of its own local parameter. The plan intersects the two and emits 2-D
strided copies ``(rows x row_bytes)``. It is pure integer arithmetic (no tensors), so it is unit-tested on CPU and
computed once per layout pair.

World layout: ranks ``0..W-1``; training rank ``r`` has tensor-parallel index ``r % tp_train``; serving rank ``r`` has
index ``r % tp_serve`` inside engine replica ``r // tp_serve``. A serving rank pulls every piece from the training rank
of its *own* training replica that holds it (itself when possible, so the common data-parallel-training case moves no
bytes over NVLink at all).

The reference's counterparts are the CUDA-IPC / NCCL refit paths and the ``nccl_reshard`` planner
(nemo_rl/models/policy/utils.py:361-549, docs/design-docs/nccl-reshard-refit.md).
"""

from __future__ import annotations

import torch
from dataclasses import dataclass, field
from typing import Optional

from rl_b200.models.config import ModelConfig
from rl_b200.models.hf_io import hf_name_map


@dataclass(frozen=True)
class CopyOp:
    src_rank: int
    dst_rank: int
    src_param: str      # trainer-side local parameter name
    dst_param: str      # engine-side local parameter name
    src_offset: int     # element offset inside the source parameter
    dst_offset: int     # element offset inside the destination parameter
    rows: int
    row_elems: int
    src_pitch: int      # elements between consecutive rows
    dst_pitch: int
    hf_name: str = ""

    @property
    def numel(self) -> int:
        return self.rows * self.row_elems


@dataclass
class RefitPlan:
    world: int
    tp_train: int
    tp_serve: int
    ops: list[CopyOp] = field(default_factory=list)

    def ops_from(self, rank: int) -> list[CopyOp]:
        return [o for o in self.ops if o.src_rank == rank]

    def ops_to(self, rank: int) -> list[CopyOp]:
        return [o for o in self.ops if o.dst_rank == rank]

    def bytes_over_link(self, rank: int, elem_bytes: int = 2) -> tuple[int, int]:
        """(bytes sent to other ranks, bytes received from other ranks) for ``rank``."""
        out = sum(o.numel for o in self.ops if o.src_rank == rank and o.dst_rank != rank) * elem_bytes
        inn = sum(o.numel for o in self.ops if o.dst_rank == rank and o.src_rank != rank) * elem_bytes
        return out, inn


def _param_shapes(cfg: ModelConfig, tp: int) -> dict[str, tuple[int, int]]:
    """(rows, cols) of every local parameter of a tensor-parallel shard, in the model's own parameter order: matrices as
    (product of the leading dimensions, last dimension), vectors as (n, 1). Read off a model built without storage, so every
    family (extra norms, latent attention, hybrid state-space blocks, stacked experts) is covered by construction."""
    from rl_b200.models.transformer import CausalLM
    from rl_b200.parallel.tensor import TP

    key = (repr(cfg), tp)
    hit = _SHAPE_CACHE.get(key)
    if hit is None:
        model = CausalLM(cfg, dtype=torch.bfloat16, device="meta", init=False, tp=TP(None, 0, tp))
        hit = {}
        for n, p in model.named_parameters():
            shp = tuple(p.shape)
            hit[n] = (shp[0], 1) if len(shp) == 1 else (int(torch.Size(shp[:-1]).numel()), shp[-1])
        _SHAPE_CACHE[key] = hit
    return dict(hit)


_SHAPE_CACHE: dict = {}


def serving_param_layout(cfg: ModelConfig, tp: int, align_elems: int = 8) -> tuple[dict[str, tuple[int, tuple[int, int]]], int]:
    """name -> (element offset in the arena, (rows, cols)) of an engine rank's weight arena, and its total elements."""
    out, off = {}, 0
    for n, shp in _param_shapes(cfg, tp).items():
        out[n] = (off, shp)
        off += -(-(shp[0] * shp[1]) // align_elems) * align_elems
    return out, off


def _pieces(cfg: ModelConfig, tp: int, rank_tp: int):
    """hf_name -> (local param, local row range or None, hf_slice or None) for one tensor-parallel index."""
    return {hf: (loc, rows, hs) for hf, loc, rows, e, hs in hf_name_map(cfg, rank_tp, tp) if e is None}


def build_refit_plan(cfg: ModelConfig, world: int, tp_train: int, tp_serve: int) -> RefitPlan:
    if cfg.is_moe:
        raise NotImplementedError("re-sharding refit of expert-parallel MoE weights: use the same layout on both sides")
    assert world % tp_train == 0 and world % tp_serve == 0
    plan = RefitPlan(world, tp_train, tp_serve)
    shapes_t, shapes_s = _param_shapes(cfg, tp_train), _param_shapes(cfg, tp_serve)
    train_pieces = [_pieces(cfg, tp_train, i) for i in range(tp_train)]
    for dst in range(world):
        need = _pieces(cfg, tp_serve, dst % tp_serve)
        replica0 = (dst // tp_train) * tp_train  # first rank of dst's training replica
        for hf, (dloc, drows, dhs) in need.items():
            d_rows_total, d_cols = shapes_s[dloc]
            d_r0 = drows[0] if drows is not None else 0
            d_nrows = (drows[1] - drows[0]) if drows is not None else d_rows_total
            # the slice of the HF tensor that dst needs, along its sharded dimension
            for ti in range(tp_train):
                sloc, srows, shs = train_pieces[ti][hf]
                s_rows_total, s_cols = shapes_t[sloc]
                s_r0 = srows[0] if srows is not None else 0
                s_nrows = (srows[1] - srows[0]) if srows is not None else s_rows_total
                if shs is None and dhs is None:
                    # replicated on both sides: one local copy from the rank's own training copy
                    if ti != dst % tp_train:
                        continue
                    plan.ops.append(CopyOp(dst, dst, sloc, dloc, s_r0 * s_cols, d_r0 * d_cols, d_nrows, d_cols, s_cols, d_cols, hf))
                    continue
                dim = (dhs or shs)[0]
                full = (shs[2] * tp_train) if shs is not None else (dhs[2] * tp_serve)
                s_lo, s_len = (shs[1], shs[2]) if shs is not None else (0, full)
                d_lo, d_len = (dhs[1], dhs[2]) if dhs is not None else (0, full)
                if shs is None and ti != dst % tp_train:
                    continue  # replicated on the training side: take it from the own rank only
                lo, hi = max(s_lo, d_lo), min(s_lo + s_len, d_lo + d_len)
                if hi <= lo:
                    continue
                src = replica0 + ti
                if dim == 0:
                    plan.ops.append(CopyOp(src, dst, sloc, dloc, (s_r0 + lo - s_lo) * s_cols, (d_r0 + lo - d_lo) * d_cols,
                                           hi - lo, d_cols, s_cols, d_cols, hf))
                else:
                    plan.ops.append(CopyOp(src, dst, sloc, dloc, s_r0 * s_cols + (lo - s_lo), d_r0 * d_cols + (lo - d_lo),
                                           d_nrows, hi - lo, s_cols, d_cols, hf))
    return plan
