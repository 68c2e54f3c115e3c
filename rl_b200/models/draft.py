"""EAGLE-3 style draft head trained beside the policy (speculative decoding: the draft proposes tokens from the policy's own
hidden states, the policy verifies them).

The draft reads, for every position t, the policy's hidden states after a few chosen layers (early / middle / late,
concatenated and mixed by ``fc``) together with the embedding of token t + 1, runs one (or more) decoder layers of the policy's
shape whose first attention sees both inputs side by side (``qkv_proj`` of width 2 * hidden), and predicts the distribution of
token t + 2 over a draft vocabulary (all policy tokens, or a frequent subset addressed through ``d2t`` offsets). Its target is
the policy's own next-token distribution at position t + 1 (soft cross-entropy, the policy detached), so the draft follows the
policy as reinforcement learning moves it.

Parameter names follow the common EAGLE-3 checkpoint layout (``fc``, ``midlayer.*``, ``norm``, ``lm_head``, ``d2t``, ``t2d``), so
a trained draft loads into serving stacks that implement EAGLE-3 and a published draft can be loaded as the starting point.

Role of nemo_rl/models/megatron/draft/eagle.py (the module), draft/hidden_capture.py (which layers are read:
``eagle3_aux_layers``) and draft/utils.py (head initialised from the policy's, HF import / export).
"""

from __future__ import annotations

import json
import os
from dataclasses import replace
from typing import Optional, Sequence

import torch
import torch.nn as nn

from rl_b200.ops import functional as F

from .config import ModelConfig
from .transformer import Attention, DenseMLP


def eagle3_aux_layers(num_layers: int) -> tuple[int, ...]:
    """Default layers whose outputs feed the draft: one early, one middle, one late (0-based, distinct, ascending)."""
    return tuple(sorted({1 if num_layers > 1 else 0, max(0, num_layers // 2 - 1), max(1 if num_layers > 1 else 0, num_layers - 4)}))


class _DraftLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device, first: bool):
        super().__init__()
        d = cfg.hidden_size
        self.cfg, self.first = cfg, first
        self.input_layernorm = nn.Parameter(torch.ones(d, dtype=dtype, device=device))
        self.self_attn = Attention(cfg, dtype, device)
        if first:   # the first layer's attention reads [normed embedding | normed hidden state]
            self.hidden_norm = nn.Parameter(torch.ones(d, dtype=dtype, device=device))
            self.self_attn.qkv_proj = nn.Parameter(torch.empty(cfg.qkv_size, 2 * d, dtype=dtype, device=device))
        self.post_attention_layernorm = nn.Parameter(torch.ones(d, dtype=dtype, device=device))
        self.mlp = DenseMLP(cfg, dtype, device)

    def forward(self, h, embeds, positions, inv_freq, cu_seqlens, max_seqlen):
        eps = self.cfg.rms_norm_eps
        if self.first:
            x = torch.cat([F.rmsnorm(embeds, self.input_layernorm, eps), F.rmsnorm(h, self.hidden_norm, eps)], dim=-1)
        else:
            x = F.rmsnorm(h, self.input_layernorm, eps)
        h = self.self_attn(x, h, positions, inv_freq, cu_seqlens, max_seqlen, 0)
        return self.mlp(F.rmsnorm(h, self.post_attention_layernorm, eps), h)


class EagleDraft(nn.Module):
    def __init__(self, policy_cfg: ModelConfig, aux_layers: Optional[Sequence[int]] = None, num_layers: int = 1,
                 draft_vocab_size: Optional[int] = None, dtype=torch.bfloat16, device="cpu"):
        super().__init__()
        c = policy_cfg
        if c.is_hybrid or c.is_mla or c.is_moe or c.sandwich_norm:
            raise NotImplementedError("the draft head is built for the Llama / Qwen dense families")
        # the draft's own layers: the policy's widths, plain attention
        self.cfg = replace(c, num_hidden_layers=int(num_layers), sliding_window=0, layer_types=None, value_head=False)
        self.aux_layers = tuple(aux_layers) if aux_layers is not None else eagle3_aux_layers(c.num_hidden_layers)
        assert all(0 <= i < c.num_hidden_layers for i in self.aux_layers)
        d = c.hidden_size
        self.draft_vocab = int(draft_vocab_size or c.vocab_size)
        self.fc = nn.Parameter(torch.empty(d, len(self.aux_layers) * d, dtype=dtype, device=device))
        self.layers = nn.ModuleList([_DraftLayer(self.cfg, dtype, device, first=(i == 0)) for i in range(int(num_layers))])
        self.norm = nn.Parameter(torch.ones(d, dtype=dtype, device=device))
        self.lm_head = nn.Parameter(torch.empty(self.draft_vocab, d, dtype=dtype, device=device))
        # draft id i stands for policy token i + d2t[i]; t2d marks the policy tokens the draft can produce
        self.register_buffer("d2t", torch.zeros(self.draft_vocab, dtype=torch.int64, device=device))
        self.register_buffer("t2d", torch.ones(c.vocab_size, dtype=torch.bool, device=device) if self.draft_vocab == c.vocab_size
                             else torch.zeros(c.vocab_size, dtype=torch.bool, device=device))
        self.reset_parameters()

    @torch.no_grad()
    def reset_parameters(self, seed: int = 0, std: float = 0.02) -> None:
        g = torch.Generator(device="cpu").manual_seed(1000003 * seed + 17)
        for n, p in self.named_parameters():
            if n.endswith("norm") or n.endswith("layernorm"):
                p.fill_(1.0)
            elif n.endswith("bias"):
                p.zero_()
            else:
                p.copy_((torch.randn(p.shape, generator=g, dtype=torch.float32) * std).to(p.dtype))

    @torch.no_grad()
    def set_vocab_subset(self, token_ids: torch.Tensor) -> None:
        """Restricts the draft vocabulary to the given policy tokens (ascending), e.g. the most frequent ones."""
        ids = torch.as_tensor(token_ids, dtype=torch.int64, device=self.d2t.device)
        assert ids.numel() == self.draft_vocab and bool((ids[1:] > ids[:-1]).all())
        self.d2t.copy_(ids - torch.arange(self.draft_vocab, device=ids.device))
        self.t2d.zero_()
        self.t2d[ids] = True

    def target_ids(self) -> torch.Tensor:
        """Policy token of every draft id."""
        return torch.arange(self.draft_vocab, device=self.d2t.device) + self.d2t

    @torch.no_grad()
    def init_head_from_policy(self, policy_head: torch.Tensor) -> None:
        """The draft's output head starts as the matching rows of the policy's."""
        self.lm_head.copy_(policy_head.detach().index_select(0, self.target_ids().to(policy_head.device)).to(self.lm_head.dtype))

    def forward(self, aux_hidden: torch.Tensor, next_embeds: torch.Tensor, positions, inv_freq, cu_seqlens, max_seqlen) -> torch.Tensor:
        """``aux_hidden`` [T, len(aux_layers) * d]: the captured hidden states, concatenated in layer order; ``next_embeds``
        [T, d]: embedding of the token that follows each position. Returns draft logits [T, draft_vocab] (fp32)."""
        h = F.linear(aux_hidden, self.fc)
        for layer in self.layers:
            h = layer(h, next_embeds, positions, inv_freq, cu_seqlens, max_seqlen)
        h = F.rmsnorm(h, self.norm, self.cfg.rms_norm_eps)
        return F.linear(h, self.lm_head).float()

    # ------------------------------------------------------------------ checkpoint names
    def _name_map(self):
        """(checkpoint name, module attribute path, row range or None)."""
        c = self.cfg
        q, kv = c.q_size, c.kv_size
        f = c.intermediate_size
        rows = [("fc.weight", "fc", None), ("norm.weight", "norm", None), ("lm_head.weight", "lm_head", None)]
        for i in range(len(self.layers)):
            hp = "midlayer" if len(self.layers) == 1 else f"midlayer.{i}"
            lp = f"layers.{i}"
            rows += [(f"{hp}.input_layernorm.weight", f"{lp}.input_layernorm", None),
                     (f"{hp}.self_attn.q_proj.weight", f"{lp}.self_attn.qkv_proj", (0, q)),
                     (f"{hp}.self_attn.k_proj.weight", f"{lp}.self_attn.qkv_proj", (q, q + kv)),
                     (f"{hp}.self_attn.v_proj.weight", f"{lp}.self_attn.qkv_proj", (q + kv, q + 2 * kv)),
                     (f"{hp}.self_attn.o_proj.weight", f"{lp}.self_attn.o_proj", None),
                     (f"{hp}.post_attention_layernorm.weight", f"{lp}.post_attention_layernorm", None),
                     (f"{hp}.mlp.gate_proj.weight", f"{lp}.mlp.gate_up_proj", (0, f)),
                     (f"{hp}.mlp.up_proj.weight", f"{lp}.mlp.gate_up_proj", (f, 2 * f)),
                     (f"{hp}.mlp.down_proj.weight", f"{lp}.mlp.down_proj", None)]
            if i == 0:
                rows.append((f"{hp}.hidden_norm.weight", f"{lp}.hidden_norm", None))
            if c.qk_norm:
                rows += [(f"{hp}.self_attn.q_norm.weight", f"{lp}.self_attn.q_norm", None),
                         (f"{hp}.self_attn.k_norm.weight", f"{lp}.self_attn.k_norm", None)]
            if c.attention_bias:
                rows += [(f"{hp}.self_attn.q_proj.bias", f"{lp}.self_attn.qkv_bias", (0, q)),
                         (f"{hp}.self_attn.k_proj.bias", f"{lp}.self_attn.qkv_bias", (q, q + kv)),
                         (f"{hp}.self_attn.v_proj.bias", f"{lp}.self_attn.qkv_bias", (q + kv, q + 2 * kv))]
        return rows

    def hf_state_dict(self) -> dict:
        params = dict(self.named_parameters())
        out = {}
        for name, loc, rows in self._name_map():
            t = params[loc].detach()
            out[name] = (t if rows is None else t[rows[0] : rows[1]]).contiguous().cpu()
        out["d2t"], out["t2d"] = self.d2t.cpu(), self.t2d.cpu()
        return out

    @torch.no_grad()
    def load_hf_state_dict(self, sd: dict, strict: bool = True) -> list[str]:
        params = dict(self.named_parameters())
        missing = []
        for name, loc, rows in self._name_map():
            src = sd.get(name)
            if src is None:
                missing.append(name)
                continue
            dst = params[loc] if rows is None else params[loc][rows[0] : rows[1]]
            if tuple(src.shape) != tuple(dst.shape):
                raise ValueError(f"{name}: checkpoint shape {tuple(src.shape)} != draft shape {tuple(dst.shape)}")
            dst.copy_(src.to(dst.dtype))
        for b in ("d2t", "t2d"):
            if b in sd:
                getattr(self, b).copy_(sd[b].to(getattr(self, b).dtype))
        if strict and missing:
            raise KeyError(f"{len(missing)} draft tensors missing, first: {missing[:4]}")
        return missing

    def save_pretrained(self, path: str) -> None:
        from safetensors.torch import save_file

        os.makedirs(path, exist_ok=True)
        save_file(self.hf_state_dict(), os.path.join(path, "model.safetensors"))
        c = self.cfg
        with open(os.path.join(path, "config.json"), "w") as f:
            json.dump(dict(architectures=["LlamaForCausalLMEagle3"], model_type="llama", hidden_size=c.hidden_size,
                           intermediate_size=c.intermediate_size, num_hidden_layers=len(self.layers), num_attention_heads=c.num_attention_heads,
                           num_key_value_heads=c.num_key_value_heads, head_dim=c.head_dim, rms_norm_eps=c.rms_norm_eps, rope_theta=c.rope_theta,
                           rope_scaling=c.rope_scaling, vocab_size=c.vocab_size, draft_vocab_size=self.draft_vocab,
                           eagle_aux_hidden_state_layer_ids=list(self.aux_layers), torch_dtype=str(self.lm_head.dtype).replace("torch.", "")), f, indent=2)

    def load_pretrained(self, path: str, strict: bool = True) -> list[str]:
        from safetensors.torch import load_file

        f = path if path.endswith(".safetensors") else os.path.join(path, "model.safetensors")
        return self.load_hf_state_dict(load_file(f), strict=strict)
