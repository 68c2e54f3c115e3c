"""Decoder-only transformer (Llama / Mistral / Qwen2 / Qwen3 / Qwen3-MoE) over *packed* token streams.

The model consumes a flat token vector ``[T]`` with ``cu_seqlens`` marking sequence boundaries (no padding tokens
ever reach a GEMM), keeps the q/k/v and gate/up projections fused, and calls the operators of
:mod:`rl_b200.ops.functional`, so that on a GPU every hot op is one of this repository's kernels. Parameters live
as views into one flat bf16 buffer (:class:`FlatParams`), which is what the sharded optimizer, the weight refit and
the generation engine address directly.

It replaces the HF modeling code + nemo-automodel wrapping that the reference's DTensor worker builds on
(nemo_rl/models/automodel/setup.py:576-878) and the mcore GPT model of its Megatron worker.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.utils.checkpoint as ckpt

from rl_b200.ops import functional as F
from rl_b200.parallel.tensor import TP, column_linear, gather_rows, row_linear, scatter_rows

from .config import ModelConfig, rope_inv_freq


def _dtype_of(name: str) -> torch.dtype:
    return {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16,
            "torch.bfloat16": torch.bfloat16, "torch.float32": torch.float32}.get(str(name), torch.bfloat16)


class FlatParams:
    """All parameters of a module tree as views of one flat buffer (plus a same-shaped gradient buffer).

    ``flat``  the parameter values (bf16 for training on GPU, fp32 for the CPU oracle); length padded to a multiple
              of ``align`` so that it splits evenly over optimizer shards.
    ``grad``  optional gradient accumulation buffer (fp32 or bf16); every parameter gets a ``main_grad`` view into
              it, and the linear / norm backward kernels accumulate into those views directly.
    """

    def __init__(self, module: nn.Module, align: int = 2048, allocator=None, include=None):
        """``allocator(numel, dtype, device) -> 1-D tensor`` lets the caller place the flat buffers (e.g. in peer-mapped
        memory); the default is an ordinary zero-filled tensor. ``include(name) -> bool`` restricts the buffer to a subset
        of the parameters (dense and expert parameters are reduced over different groups and live in two buffers)."""
        self._allocator = allocator
        params = [(n, p) for n, p in module.named_parameters() if include is None or include(n)]
        self.names = [n for n, _ in params]
        self.shapes = [tuple(p.shape) for _, p in params]
        self.numels = [p.numel() for _, p in params]
        # every tensor starts on a 16-byte boundary (TMA / vector loads)
        self.offsets = []
        off = 0
        for n in self.numels:
            self.offsets.append(off)
            off += -(-n // 8) * 8
        self.numel = off
        self.padded = -(-off // align) * align
        p0 = params[0][1]
        if allocator is not None:
            self.flat = allocator(self.padded, p0.dtype, p0.device)
            self.flat.zero_()
        else:
            self.flat = torch.zeros(self.padded, dtype=p0.dtype, device=p0.device)
        for (name, p), o, n in zip(params, self.offsets, self.numels):
            self.flat[o : o + n].copy_(p.data.reshape(-1))
            p.data = self.flat[o : o + n].view(p.shape)
        self.params = [p for _, p in params]
        self.grad: Optional[torch.Tensor] = None

    def attach_grad_buffer(self, dtype: torch.dtype = torch.float32, allocator=None) -> torch.Tensor:
        if allocator is not None:
            self.grad = allocator(self.padded, dtype, self.flat.device)
            self.grad.zero_()
        else:
            self.grad = torch.zeros(self.padded, dtype=dtype, device=self.flat.device)
        for p, o, n in zip(self.params, self.offsets, self.numels):
            p.main_grad = self.grad[o : o + n].view(p.shape)
        return self.grad

    def drop_grad_buffer(self) -> None:
        self.grad = None
        for p in self.params:
            if hasattr(p, "main_grad"):
                del p.main_grad

    def fold_autograd_grads(self) -> None:
        """Adds any ``.grad`` that autograd produced (ops without a fused accumulate path) into ``main_grad``."""
        for p in self.params:
            if p.grad is not None:
                if getattr(p, "main_grad", None) is not None:
                    p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                    p.grad = None

    def named_slices(self):
        for n, o, k, s in zip(self.names, self.offsets, self.numels, self.shapes):
            yield n, o, k, s


class LoRA(nn.Module):
    """Low-rank adapters of one fused projection. The fused weight [N_total, K] is a stack of HF projections (segments);
    every enabled segment s gets its own pair A_s [r, K], B_s [n_s, r] (PEFT-compatible), stored as ``lora_A`` [S*r, K] and
    ``lora_B`` [N_total, r] (rows of disabled segments stay zero and frozen through a mask). ``delta(x)`` returns
    scale * B_s A_s x per segment, concatenated along the output dimension
    (LoRAConfig: nemo_rl/models/policy/__init__.py:95-105)."""

    def __init__(self, segments: list[tuple[str, int]], in_features: int, cfg: dict, dtype, device):
        super().__init__()
        r = int(cfg.get("dim", 8))
        self.r, self.scale = r, float(cfg.get("alpha", 32)) / r
        targets = cfg.get("target_modules") or []
        exclude = cfg.get("exclude_modules") or []
        self.segments = segments
        self.enabled = [(not targets or n in targets or "all-linear" in targets) and n not in exclude for n, _ in segments]
        S, N = len(segments), sum(n for _, n in segments)
        self.lora_A = nn.Parameter(torch.empty(S * r, in_features, dtype=dtype, device=device))
        self.lora_B = nn.Parameter(torch.zeros(N, r, dtype=dtype, device=device))
        self.active = True

    @torch.no_grad()
    def reset(self, gen: torch.Generator) -> None:
        a = torch.randn(self.lora_A.shape, generator=gen, device=self.lora_A.device, dtype=torch.float32) / math.sqrt(self.lora_A.shape[1])
        self.lora_A.copy_(a.to(self.lora_A.dtype))
        self.lora_B.zero_()

    def delta(self, x: torch.Tensor) -> Optional[torch.Tensor]:
        if not self.active or not any(self.enabled):
            return None
        t = F.linear(x, self.lora_A)  # [T, S*r]
        outs, row = [], 0
        for s, (name, n) in enumerate(self.segments):
            if self.enabled[s]:
                outs.append(F.linear(t[:, s * self.r : (s + 1) * self.r].contiguous(), self.lora_B[row : row + n]) * self.scale)
            else:
                outs.append(torch.zeros((x.shape[0], n), dtype=x.dtype, device=x.device))
            row += n
        return outs[0] if len(outs) == 1 else torch.cat(outs, dim=1)


class Attention(nn.Module):
    """Fused-QKV attention. With tensor parallelism this rank holds ``Hq/tp`` query and ``Hkv/tp`` key/value heads:
    ``qkv_proj`` is column-parallel (rows = local q, k, v heads), ``o_proj`` row-parallel."""

    def __init__(self, cfg: ModelConfig, dtype, device, tp: Optional[TP] = None, cp=None, lora: Optional[dict] = None):
        super().__init__()
        self.cfg = cfg
        self.tp = tp or TP()
        self.cp = cp if (cp is not None and cp.world > 1) else None
        self.qkv_lora = self.o_lora = None
        if lora:
            assert self.tp.world == 1, "LoRA adapters are not tensor parallel"
            self.qkv_lora = LoRA([("q_proj", cfg.q_size), ("k_proj", cfg.kv_size), ("v_proj", cfg.kv_size)], cfg.hidden_size, lora, dtype, device)
            self.o_lora = LoRA([("o_proj", cfg.hidden_size)], cfg.q_size, lora, dtype, device)
        assert self.cp is None or self.tp.world == 1, "context parallelism and tensor parallelism are not combined"
        w = self.tp.world
        assert cfg.num_attention_heads % w == 0 and cfg.num_key_value_heads % w == 0, "heads must divide by the tensor-parallel size"
        self.hq, self.hkv = cfg.num_attention_heads // w, cfg.num_key_value_heads // w
        self.q_local, self.kv_local = self.hq * cfg.head_dim, self.hkv * cfg.head_dim
        d = cfg.hidden_size
        qkv = self.q_local + 2 * self.kv_local
        self.qkv_proj = nn.Parameter(torch.empty(qkv, d, dtype=dtype, device=device))
        self.qkv_bias = nn.Parameter(torch.zeros(qkv, dtype=dtype, device=device)) if cfg.attention_bias else None
        self.o_proj = nn.Parameter(torch.empty(d, self.q_local, dtype=dtype, device=device))
        if cfg.qk_norm:
            self.q_norm = nn.Parameter(torch.ones(cfg.head_dim, dtype=dtype, device=device))
            self.k_norm = nn.Parameter(torch.ones(cfg.head_dim, dtype=dtype, device=device))

    def project_qkv(self, x, positions, inv_freq, apply_rope: bool = True):
        """x [T, d] -> fused [T, (Hq+2Hkv)*D] with q/k normalised (Qwen3) and rotated (``apply_rope=False``: the caller
        rotates, e.g. fused with the KV-cache write of the generation engine)."""
        c = self.cfg
        qkv = column_linear(x, self.qkv_proj, self.qkv_bias, self.tp)
        if self.qkv_lora is not None:
            d = self.qkv_lora.delta(x)
            if d is not None:
                qkv = qkv + d
        if c.qk_norm:
            qkv = F.head_rmsnorm(qkv, self.q_norm, 0, self.hq, c.head_dim, c.rms_norm_eps)
            qkv = F.head_rmsnorm(qkv, self.k_norm, self.q_local, self.hkv, c.head_dim, c.rms_norm_eps)
        if not apply_rope:
            return qkv
        return F.rope(qkv, positions, inv_freq, self.hq + self.hkv, c.head_dim)

    def forward(self, x, residual, positions, inv_freq, cu_seqlens, max_seqlen, window: int = 0):
        c = self.cfg
        if self.cp is not None:
            assert not window and c.attn_scale is None, "context parallelism: no sliding windows / custom attention scale"
            from rl_b200.parallel.context import cp_attention_varlen

            T = positions.numel()
            qkv = self.project_qkv(x, positions[self.cp.local_index(T, positions.device)], inv_freq)
            a = cp_attention_varlen(qkv, cu_seqlens, self.cp, self.hq, self.hkv, c.head_dim, total_rows=T)
            return F.linear(a, self.o_proj, None, residual)
        qkv = self.project_qkv(x, positions, inv_freq)
        a = F.attention_varlen(qkv, cu_seqlens, max_seqlen, self.hq, self.hkv, c.head_dim, scale=c.attn_scale, window=window)
        return self.project_out(a, residual)

    def project_out(self, a, residual):
        y = row_linear(a, self.o_proj, residual, self.tp)
        if self.o_lora is not None:
            d = self.o_lora.delta(a)
            if d is not None:
                y = y + d
        return y


def _rope_interleaved(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, interleave: bool) -> torch.Tensor:
    """Rotary embedding of ``x`` [T, H, R]. ``interleave``: the R dimensions are stored as (even, odd) pairs and are first
    regrouped into halves (DeepSeek checkpoints); the rotation itself is the half-split form."""
    T, H, R = x.shape
    if interleave:
        x = x.reshape(T, H, R // 2, 2).transpose(2, 3).reshape(T, H, R)
    ang = positions.float()[:, None] * inv_freq.float()[None, :]            # [T, R / 2]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    x1, x2 = x[..., : R // 2].float(), x[..., R // 2 :].float()
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(x.dtype)


class MLAAttention(nn.Module):
    """Multi-head latent attention (DeepSeek-V2 / V3): queries go through a low-rank bottleneck, keys and values are
    decompressed per head from one shared latent of width ``kv_lora_rank``, and positions enter through a small decoupled
    rotary part (``qk_rope_head_dim`` dimensions, one rotary key shared by all heads).

    For the attention kernels and the generation engine's paged cache the result is laid out like ordinary attention with
    ``H`` query and ``H`` key / value heads of ``qk_nope_head_dim + qk_rope_head_dim`` dimensions; values are zero-padded to
    that width and the padding is dropped before ``o_proj``. (The engine therefore caches decompressed keys and values, not
    the latent: simple, at the cost of the memory MLA was designed to save.) Not tensor parallel."""

    def __init__(self, cfg: ModelConfig, dtype, device, tp: Optional[TP] = None, cp=None, lora: Optional[dict] = None):
        super().__init__()
        self.cfg, self.tp = cfg, tp or TP()
        assert self.tp.world == 1 and (cp is None or cp.world == 1) and not lora, "MLA: no tensor / context parallelism, no LoRA"
        self.cp = None
        self.qkv_lora = self.o_lora = None
        d, H = cfg.hidden_size, cfg.num_attention_heads
        self.hq = self.hkv = H
        self.nope, self.rope, self.vd = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim
        self.dq = self.nope + self.rope
        assert cfg.head_dim == self.dq and self.vd <= self.dq
        self.q_local = self.kv_local = H * self.dq
        P = lambda *shape: nn.Parameter(torch.empty(*shape, dtype=dtype, device=device))   # noqa: E731
        if cfg.q_lora_rank:
            self.q_a_proj, self.q_b_proj = P(cfg.q_lora_rank, d), P(H * self.dq, cfg.q_lora_rank)
            self.q_a_layernorm = nn.Parameter(torch.ones(cfg.q_lora_rank, dtype=dtype, device=device))
        else:
            self.q_proj = P(H * self.dq, d)
        self.kv_a_proj = P(cfg.kv_lora_rank + self.rope, d)
        self.kv_a_layernorm = nn.Parameter(torch.ones(cfg.kv_lora_rank, dtype=dtype, device=device))
        self.kv_b_proj = P(H * (self.nope + self.vd), cfg.kv_lora_rank)
        self.o_proj = P(d, H * self.vd)
        self.qkv_bias = None

    def project_qkv(self, x, positions, inv_freq, apply_rope: bool = True):
        """x [T, d] -> fused [T, 3 * H * dq] = [q | k | v (zero-padded)], already rotated (the rotary part is rotated here
        whatever ``apply_rope`` says: callers that rotate themselves are handed zero frequencies for these layers)."""
        c = self.cfg
        T, H = x.shape[0], self.hq
        eps = c.rms_norm_eps
        if c.q_lora_rank:
            q = F.linear(F.rmsnorm(F.linear(x, self.q_a_proj), self.q_a_layernorm, eps), self.q_b_proj)
        else:
            q = F.linear(x, self.q_proj)
        q = q.reshape(T, H, self.dq)
        ckv = F.linear(x, self.kv_a_proj)
        lat, k_rot = ckv[:, : c.kv_lora_rank], ckv[:, c.kv_lora_rank :]
        kv = F.linear(F.rmsnorm(lat.contiguous(), self.kv_a_layernorm, eps), self.kv_b_proj).reshape(T, H, self.nope + self.vd)
        q_rot = _rope_interleaved(q[..., self.nope :], positions, inv_freq, c.rope_interleave)
        k_rot = _rope_interleaved(k_rot.reshape(T, 1, self.rope), positions, inv_freq, c.rope_interleave).expand(T, H, self.rope)
        qf = torch.cat([q[..., : self.nope], q_rot], dim=-1)
        kf = torch.cat([kv[..., : self.nope], k_rot], dim=-1)
        vf = torch.nn.functional.pad(kv[..., self.nope :], (0, self.dq - self.vd))
        return torch.cat([qf.reshape(T, -1), kf.reshape(T, -1), vf.reshape(T, -1)], dim=1)

    def forward(self, x, residual, positions, inv_freq, cu_seqlens, max_seqlen, window: int = 0):
        c = self.cfg
        qkv = self.project_qkv(x, positions, inv_freq)
        a = F.attention_varlen(qkv, cu_seqlens, max_seqlen, self.hq, self.hkv, self.dq, scale=c.attn_scale, window=window)
        return self.project_out(a, residual)

    def project_out(self, a, residual):
        T = a.shape[0]
        a = a.reshape(T, self.hq, self.dq)[..., : self.vd].reshape(T, self.hq * self.vd)
        return F.linear(a.contiguous(), self.o_proj, None, residual)


class DenseMLP(nn.Module):
    """SwiGLU MLP; ``gate_up_proj`` rows are [local gate | local up] (column-parallel), ``down_proj`` row-parallel."""

    def __init__(self, cfg: ModelConfig, dtype, device, tp: Optional[TP] = None, lora: Optional[dict] = None,
                 intermediate_size: Optional[int] = None):
        super().__init__()
        self.tp = tp or TP()
        inter = intermediate_size or cfg.intermediate_size
        assert inter % self.tp.world == 0
        d, f = cfg.hidden_size, inter // self.tp.world
        self.gated = cfg.mlp_gated
        if cfg.mlp_bias:
            raise NotImplementedError("MLP biases are not supported")
        if self.gated:
            self.gate_up_proj = nn.Parameter(torch.empty(2 * f, d, dtype=dtype, device=device))
        else:   # down(act(up(x))): Nemotron-H
            self.up_proj = nn.Parameter(torch.empty(f, d, dtype=dtype, device=device))
        self.down_proj = nn.Parameter(torch.empty(d, f, dtype=dtype, device=device))
        self.act = cfg.hidden_act
        self.gate_up_lora = self.down_lora = None
        if lora and not self.gated:
            raise NotImplementedError("LoRA adapters on the non-gated MLP")
        if lora:
            assert self.tp.world == 1, "LoRA adapters are not tensor parallel"
            self.gate_up_lora = LoRA([("gate_proj", f), ("up_proj", f)], d, lora, dtype, device)
            self.down_lora = LoRA([("down_proj", d)], f, lora, dtype, device)

    def forward(self, x, residual):
        if not self.gated:
            return row_linear(F.plain_act(column_linear(x, self.up_proj, None, self.tp), self.act), self.down_proj, residual, self.tp)
        h = column_linear(x, self.gate_up_proj, None, self.tp)
        if self.gate_up_lora is not None:
            dl = self.gate_up_lora.delta(x)
            if dl is not None:
                h = h + dl
        a = F.gated_act(h, self.act)
        y = row_linear(a, self.down_proj, residual, self.tp)
        if self.down_lora is not None:
            dl = self.down_lora.delta(a)
            if dl is not None:
                y = y + dl
        return y


class DecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device, tp: Optional[TP] = None, ep=None, cp=None, lora: Optional[dict] = None,
                 layer_idx: int = 0):
        super().__init__()
        self.cfg = cfg
        d = cfg.hidden_size
        self.layer_idx = layer_idx
        self.window = cfg.sliding_window if cfg.layer_is_sliding(layer_idx) else 0
        if cfg.sandwich_norm:   # Gemma: the block outputs are normalised too, before they join the residual stream
            self.pre_feedforward_layernorm = nn.Parameter(torch.ones(d, dtype=dtype, device=device))
            self.post_feedforward_layernorm = nn.Parameter(torch.ones(d, dtype=dtype, device=device))
        self.input_layernorm = nn.Parameter(torch.ones(d, dtype=dtype, device=device))
        self.self_attn = (MLAAttention if cfg.is_mla else Attention)(cfg, dtype, device, tp, cp, lora)
        self.post_attention_layernorm = nn.Parameter(torch.ones(d, dtype=dtype, device=device))
        if cfg.layer_is_moe(layer_idx):
            from .moe import MoEMLP

            assert tp is None or tp.world == 1, "MoE layers shard experts (ep), not tensors"
            self.mlp = MoEMLP(cfg, dtype, device, ep=ep)
        else:
            self.mlp = DenseMLP(cfg, dtype, device, tp, lora)

    def forward(self, h, positions, inv_freq, cu_seqlens, max_seqlen):
        """``inv_freq``: the model's RoPE frequencies, or a pair (global, local) when sliding-window layers rotate with
        their own base."""
        eps = self.cfg.rms_norm_eps
        if isinstance(inv_freq, tuple):
            inv_freq = inv_freq[1] if self.window else inv_freq[0]
        if self.cfg.sandwich_norm:
            a = self.self_attn(F.rmsnorm(h, self.input_layernorm, eps), None, positions, inv_freq, cu_seqlens, max_seqlen, self.window)
            h = h + F.rmsnorm(a, self.post_attention_layernorm, eps)
            m = self.mlp(F.rmsnorm(h, self.pre_feedforward_layernorm, eps), None)
            return h + F.rmsnorm(m, self.post_feedforward_layernorm, eps)
        h = self.self_attn(F.rmsnorm(h, self.input_layernorm, eps), h, positions, inv_freq, cu_seqlens, max_seqlen, self.window)
        h = self.mlp(F.rmsnorm(h, self.post_attention_layernorm, eps), h)
        return h

    def tail(self, h, a):
        """From the attention output ``a`` (before o_proj) to the layer's output; used by the generation engine, whose
        attention runs over its paged cache."""
        eps = self.cfg.rms_norm_eps
        if self.cfg.sandwich_norm:
            h = h + F.rmsnorm(self.self_attn.project_out(a, None), self.post_attention_layernorm, eps)
            m = self.mlp(F.rmsnorm(h, self.pre_feedforward_layernorm, eps), None)
            return h + F.rmsnorm(m, self.post_feedforward_layernorm, eps)
        h = self.self_attn.project_out(a, h)
        return self.mlp(F.rmsnorm(h, self.post_attention_layernorm, eps), h)


class HybridBlock(nn.Module):
    """One layer of a hybrid model (Nemotron-H): RMSNorm, then ONE mixer -- a Mamba-2 state-space mixer, attention
    (no positional rotation), a plain MLP or a mixture of experts -- added to the residual stream. Only the MLP mixers are
    tensor parallel (the plan of nemo_rl/models/dtensor/parallelize.py:465); the others are replicated over the group."""

    def __init__(self, cfg: ModelConfig, dtype, device, tp: Optional[TP] = None, ep=None, cp=None, lora: Optional[dict] = None,
                 layer_idx: int = 0):
        super().__init__()
        self.cfg, self.layer_idx, self.window = cfg, layer_idx, 0
        self.kind = cfg.block_type(layer_idx)
        assert cp is None or cp.world == 1, "context parallelism is not available for hybrid state-space models"
        assert not lora, "LoRA adapters are not available for hybrid state-space models"
        self.norm = nn.Parameter(torch.ones(cfg.hidden_size, dtype=dtype, device=device))
        # the mixer sits under the name its kind has in the other families (checkpoints call all of them "mixer")
        self.mamba = self.self_attn = self.mlp = None
        if self.kind == "mamba":
            from .mamba import Mamba2Mixer

            self.mamba = Mamba2Mixer(cfg, dtype, device)
        elif self.kind == "attention":
            self.self_attn = Attention(cfg, dtype, device, None, None, None)
        elif self.kind == "mlp":
            self.mlp = DenseMLP(cfg, dtype, device, tp)
        elif self.kind == "moe":
            from .moe import MoEMLP

            self.mlp = MoEMLP(cfg, dtype, device, ep=ep)
        else:
            raise ValueError(f"unknown block type {self.kind!r}")

    @property
    def input_layernorm(self):   # the generation engine's attention path reads the pre-mixer norm under this name
        return self.norm

    def tail(self, h, a):
        """Attention blocks only: from the attention output (before o_proj) to the block's output."""
        return self.self_attn.project_out(a, h)

    def forward(self, h, positions, inv_freq, cu_seqlens, max_seqlen):
        x = F.rmsnorm(h, self.norm, self.cfg.rms_norm_eps)
        if self.kind == "mamba":
            return h + self.mamba(x, cu_seqlens, max_seqlen)
        if self.kind == "attention":
            return self.self_attn(x, h, positions, inv_freq, cu_seqlens, max_seqlen, 0)
        return self.mlp(x, h)


@dataclass
class PackedBatch:
    """A packed micro-batch: ``input_ids`` [T], ``positions`` [T], ``cu_seqlens`` [B+1] (int32), ``max_seqlen``."""

    input_ids: torch.Tensor
    positions: torch.Tensor
    cu_seqlens: torch.Tensor
    max_seqlen: int
    num_real_tokens: Optional[int] = None  # set when a dummy tail sequence pads the stream (see pad_to_multiple)

    def pad_to_multiple(self, m: int, pad_id: int = 0) -> "PackedBatch":
        """Appends one dummy sequence of pad tokens so that the token count divides by ``m`` (sequence-parallel rows
        must split evenly over the tensor-parallel ranks). Per-token outputs keep the real tokens first."""
        T = int(self.input_ids.numel())
        r = (-T) % m
        if r == 0:
            return self
        dev = self.input_ids.device
        ids = torch.cat([self.input_ids, torch.full((r,), pad_id, dtype=self.input_ids.dtype, device=dev)])
        pos = torch.cat([self.positions, torch.arange(r, dtype=self.positions.dtype, device=dev)])
        cu = torch.cat([self.cu_seqlens, torch.tensor([T + r], dtype=self.cu_seqlens.dtype, device=dev)])
        return PackedBatch(ids, pos, cu, max(self.max_seqlen, r), num_real_tokens=T)

    @staticmethod
    def from_padded(input_ids: torch.Tensor, lengths: torch.Tensor) -> "PackedBatch":
        """[B, S] right-padded ids + lengths [B] -> packed stream (pads dropped)."""
        B, S = input_ids.shape
        lengths = lengths.to(input_ids.device).long().clamp(max=S)
        ar = torch.arange(S, device=input_ids.device)
        keep = ar[None, :] < lengths[:, None]
        ids = input_ids[keep]
        pos = ar[None, :].expand(B, S)[keep]
        cu = torch.zeros(B + 1, dtype=torch.int32, device=input_ids.device)
        cu[1:] = lengths.cumsum(0).to(torch.int32)
        return PackedBatch(ids.contiguous(), pos.to(torch.int32).contiguous(), cu, int(lengths.max().item()) if B else 0)

    def unpack(self, flat: torch.Tensor, S: int, fill=0.0) -> torch.Tensor:
        """[T, ...] packed values -> [B, S, ...] right-padded."""
        cu = self.cu_seqlens
        if self.num_real_tokens is not None:  # drop the dummy tail sequence
            cu, flat = cu[:-1], flat[: self.num_real_tokens]
        B = cu.numel() - 1
        lengths = (cu[1:] - cu[:-1]).long()
        out = flat.new_full((B, S) + tuple(flat.shape[1:]), fill)
        ar = torch.arange(S, device=flat.device)
        keep = ar[None, :] < lengths[:, None]
        out[keep] = flat
        return out


class CausalLM(nn.Module):
    """Packed-sequence causal language model with HF-compatible weights (see :mod:`rl_b200.models.hf_io`).

    Model parallelism: ``tp`` shards attention heads, MLP columns and the output vocabulary over a tensor-parallel group
    (activations between blocks are sequence parallel when ``tp.sequence_parallel``); ``ep`` shards MoE experts;
    ``pp_rank`` / ``pp_size`` keep a contiguous slice of the layers on this rank (embedding on the first stage, final
    norm and output head on the last). ``vpp`` > 1 interleaves: the layers are cut into ``pp_size * vpp`` runs, run
    ``c * pp_size + pp_rank`` is this rank's chunk ``c`` (``self.layers`` holds the chunks one after another,
    ``self.layer_ids`` their global indices) and ``active_chunk`` selects the chunk a forward call runs."""

    def __init__(self, cfg: ModelConfig, dtype: Optional[torch.dtype] = None, device="cpu", init: bool = True,
                 seed: int = 0, activation_checkpointing: bool = False, tp: Optional[TP] = None, ep=None,
                 pp_rank: int = 0, pp_size: int = 1, cp=None, lora: Optional[dict] = None, vpp: int = 1):
        super().__init__()
        self.cfg = cfg
        self.lora_cfg = dict(lora) if (lora and lora.get("enabled", True)) else None
        dtype = dtype or _dtype_of(cfg.torch_dtype)
        self.dtype = dtype
        self.tp = tp or TP()
        self.ep = ep
        self.cp = cp if (cp is not None and cp.world > 1) else None
        self.pp_rank, self.pp_size = pp_rank, pp_size
        L = cfg.num_hidden_layers
        self.vpp = max(1, int(vpp)) if pp_size > 1 else 1
        per = -(-L // (pp_size * self.vpp))
        self.layer_ids, self.chunk_bounds = [], []      # global index of local layer j; [lo, hi) local range of chunk c
        for c in range(self.vpp):
            lo = (c * pp_size + pp_rank) * per
            ids = list(range(lo, max(lo, min(L, lo + per))))
            self.chunk_bounds.append((len(self.layer_ids), len(self.layer_ids) + len(ids)))
            self.layer_ids += ids
        self.layer_offset = self.layer_ids[0] if self.layer_ids else min(L, pp_rank * per)   # (meaningful when vpp == 1)
        self.active_chunk: Optional[int] = None
        n_local = len(self.layer_ids)
        self.first_stage, self.last_stage = pp_rank == 0, pp_rank == pp_size - 1
        d = cfg.hidden_size
        tpw = self.tp.world
        assert cfg.vocab_size % tpw == 0, "vocabulary must divide by the tensor-parallel size"
        self.vocab_local = cfg.vocab_size // tpw
        self.vocab_start = self.tp.rank * self.vocab_local
        tied = cfg.tie_word_embeddings and not cfg.value_head
        if self.first_stage or (self.last_stage and tied):
            self.embed_tokens = nn.Parameter(torch.empty(cfg.vocab_size, d, dtype=dtype, device=device))
        else:
            self.embed_tokens = None
        block = HybridBlock if cfg.is_hybrid else DecoderLayer
        if cfg.is_hybrid and self.tp.sequence_parallel:
            raise NotImplementedError("sequence parallelism is not available for hybrid state-space models")
        self.layers = nn.ModuleList([block(cfg, dtype, device, self.tp, ep, self.cp, self.lora_cfg, layer_idx=self.layer_ids[i])
                                     for i in range(n_local)])
        self.lm_head = None
        if self.last_stage:
            self.norm = nn.Parameter(torch.ones(d, dtype=dtype, device=device))
            if cfg.value_head:
                self.score = nn.Parameter(torch.empty(8, d, dtype=dtype, device=device))  # row 0 is the head; 8 rows keep TMA alignment
            elif not tied:
                self.lm_head = nn.Parameter(torch.empty(self.vocab_local, d, dtype=dtype, device=device))
        else:
            self.norm = None
        self.register_buffer("inv_freq", rope_inv_freq(cfg, device), persistent=False)
        if cfg.rope_local_theta:   # sliding-window layers rotate with their own base and no long-context scaling
            from dataclasses import replace

            self.register_buffer("inv_freq_local", rope_inv_freq(replace(cfg, rope_theta=cfg.rope_local_theta, rope_scaling=None), device),
                                 persistent=False)
        else:
            self.inv_freq_local = None
        if cfg.final_logit_softcap:
            raise NotImplementedError("final logit soft-capping (Gemma 2) is not supported by the fused log-probability paths")
        self.activation_checkpointing = activation_checkpointing
        if init:
            self.reset_parameters(seed)
        self.flat: Optional[FlatParams] = None
        # fully sharded parameters (rl_b200/parallel/fsdp.py): when set, every unit of the model (embedding, each layer,
        # the head) runs through ``sharder.run`` which gathers its parameters for the duration of the call
        self.sharder = None
        # draft-head training (rl_b200/models/draft.py): when set, the outputs of these layers (global indices), the token
        # embeddings ("embeds") and the normed final hidden states ("final") of the last forward are kept in ``captured``
        self.capture_layers: Optional[tuple] = None
        self.captured: dict = {}

    # ------------------------------------------------------------------ parameters
    _TP_SHARDED = ("qkv_proj", "qkv_bias", "o_proj", "gate_up_proj", "up_proj", "down_proj", "lm_head")

    def is_tp_sharded(self, name: str) -> bool:
        """Whether parameter ``name`` holds a tensor-parallel shard (False: replicated over the tp group)."""
        if self.tp.world == 1:
            return False
        leaf = name.rsplit(".", 1)[-1]
        if self.cfg.is_hybrid:   # only the plain MLP blocks and the output head are sharded
            if leaf == "lm_head":
                return True
            if leaf not in ("up_proj", "down_proj") or ".mlp." not in name or "shared_experts" in name:
                return False
            li = self.layer_ids[int(name.split(".")[1])]
            return self.cfg.block_type(li) == "mlp"
        return leaf in self._TP_SHARDED and ".mlp.router" not in name and not (self.cfg.is_moe and ".mlp." in name)

    @torch.no_grad()
    def reset_parameters(self, seed: int = 0, std: float = 0.02) -> None:
        """Normal(0, 0.02) weights (HF's default initializer range), ones for norms, zeros for biases.

        Every logical (HuggingFace-named) tensor is drawn from its own generator seeded by ``seed`` and the tensor's name,
        and each rank keeps its slice: the model is the same whatever the tensor / pipeline / expert layout is."""
        import zlib

        from .hf_io import iter_hf_shards, hf_full_shape

        for name, p in self.named_parameters():
            if name.endswith("norm") or name.endswith("layernorm"):
                p.fill_(1.0)
            elif name.endswith("bias"):
                p.zero_()
        for name, mod in self.named_modules():
            if isinstance(mod, LoRA):
                g = torch.Generator(device=mod.lora_A.device)
                g.manual_seed((seed * 1000003 + zlib.crc32(name.encode())) & 0x7FFFFFFFFFFFFFFF)
                mod.reset(g)
        for mname, mod in self.named_modules():
            if hasattr(mod, "reset_special"):   # state-space mixers: decay rates, step sizes, skip weights
                g = torch.Generator(device=mod.dt_bias.device)
                g.manual_seed((seed * 1000003 + zlib.crc32(mname.encode())) & 0x7FFFFFFFFFFFFFFF)
                mod.reset_special(g)
        for hf, dst, hs in iter_hf_shards(self):
            if hf.endswith("norm.weight") or hf.endswith("layernorm.weight") or hf.endswith("norm_f.weight") or hf.endswith(".bias"):
                continue
            if hf.endswith(".A_log") or hf.endswith(".D") or hf.endswith(".dt_bias"):
                continue
            if hf.endswith("e_score_correction_bias"):
                dst.zero_()
                continue
            g = torch.Generator(device=dst.device)
            g.manual_seed((seed * 1000003 + zlib.crc32(hf.encode())) & 0x7FFFFFFFFFFFFFFF)
            full = hf_full_shape(tuple(dst.shape), hs, self.tp.world)
            rows, cols = full[0], (full[1] if len(full) > 1 else 1)
            r0, r1 = (hs[1], hs[1] + hs[2]) if hs is not None and hs[0] == 0 else (0, rows)
            c0, c1 = (hs[1], hs[1] + hs[2]) if hs is not None and hs[0] == 1 else (0, cols)
            # rows are generated in order in bounded fp32 chunks; only this rank's slice is kept
            step = max(1, (1 << 26) // max(1, cols))
            d2 = dst.view(dst.shape[0], -1)
            cols = d2.shape[1] if hs is None else cols      # (3-D tensors such as the depth-wise conv: all trailing dimensions)
            c1 = cols if hs is None else c1
            for s0 in range(0, r1, step):
                e0 = min(rows, s0 + step)
                blk = torch.randn((e0 - s0, cols), generator=g, device=dst.device, dtype=torch.float32) * std
                lo, hi = max(s0, r0), min(e0, r1)
                if hi > lo:
                    d2[lo - r0 : hi - r0].copy_(blk[lo - s0 : hi - s0, c0:c1].to(dst.dtype))
        if self.cfg.value_head and self.last_stage:
            self.score[1:].zero_()

    def flatten_parameters(self, align: int = 2048, allocator=None, include=None) -> FlatParams:
        fl = FlatParams(self, align, allocator, include)
        if include is None or self.flat is None:
            self.flat = fl
        return fl

    @staticmethod
    def is_lora_param(name: str) -> bool:
        return name.endswith(".lora_A") or name.endswith(".lora_B")

    def set_adapters(self, active: bool) -> None:
        """Switches every LoRA adapter on or off (off = the frozen base model, i.e. the reference policy)."""
        for mod in self.modules():
            if isinstance(mod, LoRA):
                mod.active = active

    @torch.no_grad()
    def merged_weight(self, fused: torch.Tensor, lora: "LoRA") -> torch.Tensor:
        """W + scale * B A for a fused projection (export / merged serving)."""
        w = fused.float().clone()
        row = 0
        for s, (_, n) in enumerate(lora.segments):
            if lora.enabled[s]:
                w[row : row + n] += lora.scale * (lora.lora_B[row : row + n].float() @ lora.lora_A[s * lora.r : (s + 1) * lora.r].float())
            row += n
        return w.to(fused.dtype)

    @staticmethod
    def is_expert_param(name: str) -> bool:
        """Expert-parallel parameters (stacked expert weights); the router is replicated like any dense parameter."""
        return name.endswith(".mlp.gate_up_proj") or name.endswith(".mlp.down_proj")

    def expert_param_names(self) -> set:
        """Names of the expert-parallel parameters of THIS model: the stacked weights of its mixture-of-experts blocks
        (a dense MLP of the same model, e.g. DeepSeek's first layers or a hybrid model's MLP blocks, is not among them)."""
        from .moe import MoEMLP

        out = set()
        for mname, mod in self.named_modules():
            if isinstance(mod, MoEMLP):
                out.update(f"{mname}.{leaf}" for leaf in ("gate_up_proj", "up_proj", "down_proj") if getattr(mod, leaf, None) is not None)
        return out

    @property
    def at_input(self) -> bool:
        """The chunk about to run starts the model (it embeds the tokens)."""
        return self.first_stage and self.active_chunk in (None, 0)

    @property
    def at_output(self) -> bool:
        """The chunk about to run ends the model (final norm, output head, loss)."""
        return self.last_stage and self.active_chunk in (None, self.vpp - 1)

    @property
    def output_weight(self) -> torch.Tensor:
        """This rank's rows of the output projection ([V/tp, d])."""
        if self.lm_head is not None:
            return self.lm_head
        if self.tp.world == 1:
            return self.embed_tokens
        return self.embed_tokens[self.vocab_start : self.vocab_start + self.vocab_local]

    # ------------------------------------------------------------------ forward
    def rope_freqs(self):
        """What the layers take as ``inv_freq``: one tensor, or (global, local) when sliding-window layers have their own."""
        return self.inv_freq if self.inv_freq_local is None else (self.inv_freq, self.inv_freq_local)

    def embed(self, batch: PackedBatch) -> torch.Tensor:
        h = self._embed(batch)
        s = self.cfg.embed_scale
        return h if s == 1.0 else h * torch.tensor(s, dtype=h.dtype, device=h.device)   # the scale is rounded to the model dtype first

    def _embed(self, batch: PackedBatch) -> torch.Tensor:
        if self.sharder is not None:
            return self.sharder.run("embed", lambda: F.embedding(batch.input_ids, self.embed_tokens))
        if self.tp.world > 1 and self.tp.sequence_parallel:
            # each rank embeds its own rows: like every replicated parameter under sequence parallelism, the table's
            # gradient is a partial sum that the worker all-reduces over the tensor-parallel group
            rows = batch.input_ids.numel() // self.tp.world
            return F.embedding(batch.input_ids[self.tp.rank * rows : (self.tp.rank + 1) * rows], self.embed_tokens)
        if self.cp is not None:
            # this rank's rows of the stream: two chunks, one early and one late (load-balanced under the causal mask)
            return F.embedding(batch.input_ids[self.cp.local_index(batch.input_ids.numel(), batch.input_ids.device)], self.embed_tokens)
        return F.embedding(batch.input_ids, self.embed_tokens)

    def run_layers(self, h: torch.Tensor, batch: PackedBatch) -> torch.Tensor:
        inv_freq = self.rope_freqs()
        if self.sharder is not None:
            for i, layer in enumerate(self.layers):
                h = self.sharder.run(f"layer{i}", lambda x, L=layer: L(x, batch.positions, inv_freq, batch.cu_seqlens, batch.max_seqlen), h)
            return h
        cap = self.capture_layers
        if cap is not None:
            self.captured = {"embeds": h}
        lo, hi = (0, len(self.layers)) if self.active_chunk is None else self.chunk_bounds[self.active_chunk]
        for i in range(lo, hi):
            layer = self.layers[i]
            if self.activation_checkpointing and torch.is_grad_enabled():
                h = ckpt.checkpoint(layer, h, batch.positions, inv_freq, batch.cu_seqlens, batch.max_seqlen, use_reentrant=False)
            else:
                h = layer(h, batch.positions, inv_freq, batch.cu_seqlens, batch.max_seqlen)
            if cap is not None and self.layer_ids[i] in cap:
                self.captured[self.layer_ids[i]] = h
        return h

    def hidden_states(self, batch: PackedBatch, h_in: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Output of this stage: the normed final hidden states on the last stage, else the residual stream handed to
        the next stage. Rows are this rank's sequence-parallel shard when ``tp.sequence_parallel``."""
        h = self.embed(batch) if self.at_input else h_in
        h = self.run_layers(h, batch)
        if self.sharder is not None:
            return self.sharder.run("head", lambda x: F.rmsnorm(x, self.norm, self.cfg.rms_norm_eps), h)
        out = F.rmsnorm(h, self.norm, self.cfg.rms_norm_eps) if self.at_output else h
        if self.capture_layers is not None and self.at_output:
            self.captured["final"] = out
        return out

    def logits(self, batch: PackedBatch, h_in: Optional[torch.Tensor] = None) -> torch.Tensor:
        """[T, V] logits in fp32 (small models, tests and the distillation / top-k paths)."""
        if self.sharder is not None:
            h = self.run_layers(self.embed(batch), batch)
            return self.sharder.run("head", lambda x: F.linear(F.rmsnorm(x, self.norm, self.cfg.rms_norm_eps), self.output_weight).float(), h)
        h = self.hidden_states(batch, h_in)
        if self.tp.world == 1:
            return F.linear(h, self.output_weight).float()
        from rl_b200.parallel.tensor import gather_cols

        return gather_cols(column_linear(h, self.output_weight, None, self.tp), self.tp).float()

    def logprobs_from_hidden(self, h: torch.Tensor, batch: PackedBatch, temperature: float = 1.0, want_entropy: bool = False):
        """``h``: normed final hidden states (this rank's rows). out[t] = log p(ids[t] | ids[<t]), 0 at sequence starts."""
        ids = batch.input_ids.long()
        T = ids.shape[0]
        starts = batch.cu_seqlens[:-1].long()
        is_start = torch.zeros(T, dtype=torch.bool, device=h.device)
        is_start[starts[starts < T]] = True
        # hidden state t predicts token t+1: every row is scored against the next token, then shifted by one
        targets = torch.roll(ids, -1)
        if self.cp is not None:
            # local rows are scored locally; the [T]-sized results are gathered (backward: each rank keeps its rows' share)
            from rl_b200.parallel.context import gather_to_stream

            lp_l, ent_l = F.lm_head_logprobs(h, self.output_weight, targets[self.cp.local_index(T, ids.device)], temperature, want_entropy)
            lp_rows = gather_to_stream(lp_l, self.cp)
            ent_rows = gather_to_stream(ent_l, self.cp) if want_entropy else None
        elif self.tp.world == 1:
            lp_rows, ent_rows = F.lm_head_logprobs(h, self.output_weight, targets, temperature, want_entropy)
        else:
            from rl_b200.parallel.vocab import vocab_parallel_logprobs

            lp_rows, ent_rows = vocab_parallel_logprobs(h, self.output_weight, targets, self.tp, self.vocab_start, temperature, want_entropy)
        valid = ~is_start[1:]
        logp = torch.zeros(T, dtype=torch.float32, device=h.device)
        logp[1:] = torch.where(valid, lp_rows[:-1], torch.zeros_like(lp_rows[:-1]))
        ent = None
        if want_entropy:
            ent = torch.zeros(T, dtype=torch.float32, device=h.device)
            ent[1:] = torch.where(valid, ent_rows[:-1], torch.zeros_like(ent_rows[:-1]))
        return logp, ent

    def next_token_logprobs(self, batch: PackedBatch, temperature: float = 1.0, want_entropy: bool = False,
                            h_in: Optional[torch.Tensor] = None):
        """Log-probability of each token given its prefix ([T] fp32, entropy [T] or None), through the fused projection +
        log-softmax (vocabulary-parallel under tensor parallelism)."""
        if self.sharder is not None:
            # the final norm and the output projection belong to one unit: they run inside one gather
            h = self.run_layers(self.embed(batch), batch)
            eps = self.cfg.rms_norm_eps
            if want_entropy:
                return self.sharder.run("head", lambda x: self.logprobs_from_hidden(F.rmsnorm(x, self.norm, eps), batch, temperature, True), h)
            return self.sharder.run("head", lambda x: self.logprobs_from_hidden(F.rmsnorm(x, self.norm, eps), batch, temperature, False)[0], h), None
        return self.logprobs_from_hidden(self.hidden_states(batch, h_in), batch, temperature, want_entropy)

    def next_token_logprobs_filtered(self, batch: PackedBatch, top_k: Optional[int], top_p: float, temperature: float = 1.0,
                                     h_in: Optional[torch.Tensor] = None, chunk_rows: int = 2048) -> torch.Tensor:
        """Log-probabilities under the sampler's *processed* distribution (temperature, then top-k / top-p): what the
        importance ratio must use when rollouts were sampled with those filters
        (nemo_rl/algorithms/logits_sampling_utils.py:112-285). The logits are materialised ``chunk_rows`` rows at a time;
        with tensor parallelism an all-to-all turns the chunk's vocabulary shards into row shards, so no rank holds
        ``[T, V]`` (nemo_rl/distributed/model_utils.py:383-510)."""
        from rl_b200.algorithms.sampling_utils import apply_top_k_top_p

        ids = batch.input_ids.long()
        T = ids.shape[0]
        targets = torch.roll(ids, -1)
        inv_t = temperature if temperature > 0 else 1.0

        def score_rows(hr, tg, w):   # rows with the whole vocabulary on this rank
            out = []
            for r0 in range(0, hr.shape[0], chunk_rows):
                z = F.linear(hr[r0 : r0 + chunk_rows], w).float() / inv_t
                z, _ = apply_top_k_top_p(z, top_k, top_p)
                lp = torch.log_softmax(z, dim=-1).gather(-1, tg[r0 : r0 + chunk_rows, None])[:, 0]
                out.append(torch.where(torch.isfinite(lp), lp, torch.full_like(lp, -1e4)))   # a token outside the kept set
            return torch.cat(out)

        if self.sharder is not None:      # fully sharded parameters: the head unit is gathered for the duration of the call
            hh = self.run_layers(self.embed(batch), batch)
            lp_rows = self.sharder.run("head", lambda x: score_rows(F.rmsnorm(x, self.norm, self.cfg.rms_norm_eps), targets, self.output_weight), hh)
        else:
            h = self.hidden_states(batch, h_in)
            if self.cp is not None:       # context parallel: every rank scores its own rows, results return to stream order
                from rl_b200.parallel.context import gather_to_stream

                lp_rows = gather_to_stream(score_rows(h, targets[self.cp.local_index(T, ids.device)], self.output_weight), self.cp)
            elif self.tp.world == 1:
                lp_rows = score_rows(h, targets, self.output_weight)
            else:                         # vocabulary parallel (with or without sequence parallelism): no [T, V] anywhere
                from rl_b200.parallel.vocab import vocab_parallel_filtered_logprobs

                lp_rows = vocab_parallel_filtered_logprobs(h, self.output_weight, targets, self.tp, temperature, top_k, top_p, chunk_rows)
        dev = lp_rows.device
        starts = batch.cu_seqlens[:-1].long()
        is_start = torch.zeros(T, dtype=torch.bool, device=dev)
        is_start[starts[starts < T]] = True
        logp = torch.zeros(T, dtype=torch.float32, device=dev)
        logp[1:] = torch.where(~is_start[1:], lp_rows[:-1], torch.zeros_like(lp_rows[:-1]))
        return logp

    def values(self, batch: PackedBatch, h_in: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Scalar head output per token [T] (critic / reward model)."""
        if self.sharder is not None:
            h = self.run_layers(self.embed(batch), batch)
            return self.sharder.run("head", lambda x: F.linear(F.rmsnorm(x, self.norm, self.cfg.rms_norm_eps), self.score).float()[:, 0], h)
        h = self.hidden_states(batch, h_in)
        v = F.linear(h, self.score).float()[:, 0]
        if self.cp is not None:
            from rl_b200.parallel.context import gather_to_stream

            return gather_to_stream(v, self.cp)
        return gather_rows(v, self.tp) if self.tp.sequence_parallel else v


def build_model(cfg: ModelConfig, device="cpu", dtype: Optional[torch.dtype] = None, seed: int = 0,
                activation_checkpointing: bool = False, init: bool = True, tp: Optional[TP] = None, ep=None,
                pp_rank: int = 0, pp_size: int = 1, cp=None, lora: Optional[dict] = None, vpp: int = 1) -> CausalLM:
    cls = CausalLM
    if cfg.vision is not None:
        from .vision import VLMCausalLM as cls
    return cls(cfg, dtype=dtype, device=device, init=init, seed=seed, activation_checkpointing=activation_checkpointing,
               tp=tp, ep=ep, pp_rank=pp_rank, pp_size=pp_size, cp=cp, lora=lora, vpp=vpp)
