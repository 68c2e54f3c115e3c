"""Architecture description for the decoder-only model families the framework trains and serves.

One dataclass covers Llama (2/3/3.1/3.2), Mistral, Qwen2/2.5, Qwen3, Qwen3-MoE and Gemma 3 (text); the differences are switches
(QKV bias, per-head q/k RMSNorm, tied embeddings, RoPE scaling, mixture-of-experts FFN; for Gemma 3: tanh-GELU gate, norms
before and after each block, scaled embeddings, sliding-window layers with their own RoPE base, a fixed attention scale). ``from_hf_dict`` reads a
HuggingFace ``config.json`` dictionary; ``PRESETS`` names the architectures used by the benchmark configs.
"""

from __future__ import annotations

import json
import math
import os
from dataclasses import asdict, dataclass, field
from typing import Any, Optional

import torch


@dataclass
class ModelConfig:
    model_type: str = "llama"
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 32
    head_dim: int = 128
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_scaling: Optional[dict] = None
    max_position_embeddings: int = 131072
    tie_word_embeddings: bool = False
    attention_bias: bool = False       # Qwen2: bias on q/k/v projections
    qk_norm: bool = False              # Qwen3: RMSNorm over head_dim on q and k before RoPE
    # mixture of experts (Qwen3-MoE): num_experts > 0 replaces the dense FFN
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True
    router_aux_loss_coef: float = 0.0
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[Any] = None
    pad_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"
    value_head: bool = False           # critic / reward model: scalar head instead of the vocabulary projection
    vision: Optional[dict] = None      # vision tower settings (models/vision.py); None: text-only model
    image_token_id: Optional[int] = None
    # Gemma 3 (nemo_rl/models/dtensor/parallelize.py:170-217 is the reference's parallel plan for this family)
    hidden_act: str = "silu"           # gate activation of the MLP: silu | gelu_pytorch_tanh
    sandwich_norm: bool = False        # RMSNorm before AND after attention / MLP (the post norms act on the block output)
    embed_scale: float = 1.0           # embeddings are multiplied by this (sqrt(hidden_size))
    norm_offset: float = 0.0           # checkpoints store RMSNorm weights as w - offset (Gemma: 1); buffers here hold w
    sliding_window: int = 0            # > 0: layers listed as "sliding_attention" see only the last `sliding_window` keys
    layer_types: Optional[list] = None  # per layer: "full_attention" | "sliding_attention"
    rope_local_theta: float = 0.0      # RoPE base of the sliding-window layers (0: same as rope_theta, scaling included)
    attn_scale: Optional[float] = None  # softmax scale when it is not head_dim ** -0.5 (query_pre_attn_scalar ** -0.5)
    final_logit_softcap: float = 0.0   # logits <- cap * tanh(logits / cap) (Gemma 2; 0: off)

    # DeepSeek-V3: multi-head latent attention and its mixture of experts
    kv_lora_rank: int = 0              # > 0: attention is MLA (keys / values decompressed from a latent of this width)
    q_lora_rank: Optional[int] = None  # low-rank query projection (None: a plain q_proj)
    qk_nope_head_dim: int = 0
    qk_rope_head_dim: int = 0
    v_head_dim: int = 0
    rope_interleave: bool = True       # checkpoints store the rotary dimensions interleaved (pairs), not split in halves
    n_shared_experts: int = 0          # dense experts every token passes through, added to the routed output
    first_k_dense_replace: int = 0     # the first k layers keep a dense MLP
    scoring_func: str = "softmax"      # router scores: softmax | sigmoid (with a per-expert selection bias)
    n_group: int = 1                   # experts are split in groups; only `topk_group` groups stay eligible per token
    topk_group: int = 1
    routed_scaling_factor: float = 1.0

    # Nemotron-H (hybrid Mamba-2 / attention / MLP / MoE; nemo_rl/models/dtensor/parallelize.py:465 is the reference's plan
    # for this family): every layer is ONE mixer behind one RMSNorm, named by ``layers_block_type``
    layers_block_type: Optional[list] = None   # per layer: "mamba" | "attention" | "mlp" | "moe"
    use_rope: bool = True              # False: attention has no positional rotation (the state-space layers carry order)
    mlp_gated: bool = True             # False: down(act(up(x))) instead of down(act(gate(x)) * up(x))
    mlp_bias: bool = False
    mamba_num_heads: int = 0
    mamba_head_dim: int = 0
    ssm_state_size: int = 0
    mamba_n_groups: int = 1
    mamba_d_conv: int = 4
    mamba_chunk_size: int = 128
    mamba_conv_bias: bool = True
    mamba_proj_bias: bool = False
    mamba_dt_limit: Optional[list] = None      # [lo, hi] clamp of the step size after softplus
    moe_latent_size: Optional[int] = None      # routed experts work in a narrower space between two shared projections
    moe_shared_expert_intermediate_size: int = 0

    @property
    def is_hybrid(self) -> bool:
        return self.layers_block_type is not None

    def block_type(self, i: int) -> str:
        """"mamba" | "attention" | "mlp" | "moe" for hybrid models, "decoder" (attention + MLP in one layer) otherwise."""
        return self.layers_block_type[i] if self.layers_block_type is not None else "decoder"

    @property
    def mamba_inner(self) -> int:
        return self.mamba_num_heads * self.mamba_head_dim

    @property
    def mamba_conv_dim(self) -> int:
        return self.mamba_inner + 2 * self.mamba_n_groups * self.ssm_state_size

    @property
    def is_mla(self) -> bool:
        return self.kv_lora_rank > 0

    def layer_is_moe(self, i: int) -> bool:
        if self.layers_block_type is not None:
            return self.layers_block_type[i] == "moe"
        return self.is_moe and i >= self.first_k_dense_replace

    def layer_is_sliding(self, i: int) -> bool:
        return bool(self.sliding_window) and self.layer_types is not None and self.layer_types[i] == "sliding_attention"

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def qkv_size(self) -> int:
        return self.q_size + 2 * self.kv_size

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    def num_parameters(self) -> int:
        d, L = self.hidden_size, self.num_hidden_layers
        if self.layers_block_type is not None:
            I, C, H = self.mamba_inner, self.mamba_conv_dim, self.mamba_num_heads
            din = self.moe_latent_size or d
            per = {"mamba": (I + C + H) * d + C * (self.mamba_d_conv + 1) + 3 * H + I + d * I,
                   "attention": d * self.qkv_size + self.q_size * d,
                   "mlp": 2 * d * self.intermediate_size,
                   "moe": self.num_experts * (2 * din * self.moe_intermediate_size + d) + 2 * d * self.moe_shared_expert_intermediate_size
                          + (2 * d * din if self.moe_latent_size else 0)}
            return sum(per[t] + d for t in self.layers_block_type) + self.vocab_size * d * (1 if self.tie_word_embeddings else 2) + d
        attn = d * self.qkv_size + self.q_size * d + (self.qkv_size if self.attention_bias else 0)
        if self.is_moe:
            ffn = self.num_experts * 3 * d * self.moe_intermediate_size + self.num_experts * d
        else:
            ffn = 3 * d * self.intermediate_size
        norms = 2 * d + (2 * self.head_dim if self.qk_norm else 0)
        emb = self.vocab_size * d * (1 if self.tie_word_embeddings else 2)
        return L * (attn + ffn + norms) + emb + d

    def to_hf_dict(self) -> dict:
        arch = {"llama": "LlamaForCausalLM", "mistral": "MistralForCausalLM", "qwen2": "Qwen2ForCausalLM",
                "qwen3": "Qwen3ForCausalLM", "qwen3_moe": "Qwen3MoeForCausalLM",
                "gemma3_text": "Gemma3ForCausalLM", "deepseek_v3": "DeepseekV3ForCausalLM",
                "nemotron_h": "NemotronHForCausalLM"}.get(self.model_type, "LlamaForCausalLM")
        d = asdict(self)
        nh = {k: d.pop(k) for k in ("layers_block_type", "use_rope", "mlp_gated", "mlp_bias", "mamba_num_heads", "mamba_head_dim", "ssm_state_size",
                                    "mamba_n_groups", "mamba_d_conv", "mamba_chunk_size", "mamba_conv_bias", "mamba_proj_bias", "mamba_dt_limit",
                                    "moe_latent_size", "moe_shared_expert_intermediate_size")}
        if self.model_type == "nemotron_h":
            pat = "".join({"mamba": "M", "attention": "*", "mlp": "-", "moe": "E"}[t] for t in nh["layers_block_type"])
            d.update(hybrid_override_pattern=pat, layers_block_type=nh["layers_block_type"], mamba_num_heads=nh["mamba_num_heads"],
                     mamba_head_dim=nh["mamba_head_dim"], ssm_state_size=nh["ssm_state_size"], n_groups=nh["mamba_n_groups"],
                     conv_kernel=nh["mamba_d_conv"], chunk_size=nh["mamba_chunk_size"], use_conv_bias=nh["mamba_conv_bias"],
                     use_bias=nh["mamba_proj_bias"], mlp_bias=nh["mlp_bias"], mlp_hidden_act=d["hidden_act"], layer_norm_epsilon=d["rms_norm_eps"],
                     time_step_limit=nh["mamba_dt_limit"] or [0.0, float("inf")], moe_latent_size=nh["moe_latent_size"],
                     moe_shared_expert_intermediate_size=nh["moe_shared_expert_intermediate_size"], n_routed_experts=self.num_experts,
                     n_shared_experts=self.n_shared_experts, n_group=self.n_group, topk_group=self.topk_group,
                     routed_scaling_factor=self.routed_scaling_factor)
        d.pop("value_head")
        d.pop("qk_norm")
        gem = {k: d.pop(k) for k in ("hidden_act", "sandwich_norm", "embed_scale", "norm_offset", "sliding_window", "layer_types",
                                     "rope_local_theta", "attn_scale", "final_logit_softcap")}
        if self.model_type == "gemma3_text":
            d.update(hidden_activation=gem["hidden_act"], sliding_window=gem["sliding_window"], layer_types=gem["layer_types"],
                     rope_local_base_freq=gem["rope_local_theta"], query_pre_attn_scalar=round(gem["attn_scale"] ** -2) if gem["attn_scale"] else self.head_dim,
                     final_logit_softcapping=gem["final_logit_softcap"] or None)
        d["architectures"] = [arch]
        if self.vision is None:
            d.pop("vision")
            d.pop("image_token_id")
        ds = {k: d.pop(k) for k in ("kv_lora_rank", "q_lora_rank", "qk_nope_head_dim", "qk_rope_head_dim", "v_head_dim", "rope_interleave",
                                    "n_shared_experts", "first_k_dense_replace", "scoring_func", "n_group", "topk_group", "routed_scaling_factor")}
        if self.model_type == "nemotron_h":
            d.update({k: ds[k] for k in ("n_shared_experts", "n_group", "topk_group", "routed_scaling_factor")})
        if self.model_type == "deepseek_v3":
            d.update(ds, n_routed_experts=self.num_experts)
            d.pop("num_experts")
            d.pop("head_dim")
        if not self.is_moe:
            for k in ("num_experts", "num_experts_per_tok", "moe_intermediate_size", "norm_topk_prob", "router_aux_loss_coef"):
                d.pop(k, None)
        return d

    @classmethod
    def from_hf_dict(cls, hf: dict, **overrides) -> "ModelConfig":
        mt = hf.get("model_type", "llama")
        if mt == "gemma3" and "text_config" in hf:      # the multimodal wrapper: the language model's settings are nested
            hf = dict(hf["text_config"], model_type="gemma3_text")
            mt = "gemma3_text"
        n_heads = hf["num_attention_heads"]
        if mt == "nemotron_h":
            hf = dict(hf)
            types = hf.get("layers_block_type")
            if types is None:    # older configs: one character per layer (M mamba, * attention, - MLP, E mixture of experts)
                types = [{"M": "mamba", "*": "attention", "-": "mlp", "E": "moe"}[ch] for ch in hf["hybrid_override_pattern"]]
            hf["layers_block_type"] = list(types)
            hf["num_hidden_layers"] = len(types)
            hf.setdefault("rms_norm_eps", hf.get("layer_norm_epsilon", 1e-5))
        cfg = cls(
            model_type=mt,
            vocab_size=hf["vocab_size"],
            hidden_size=hf["hidden_size"],
            intermediate_size=hf.get("intermediate_size", 0),
            num_hidden_layers=hf["num_hidden_layers"],
            num_attention_heads=n_heads,
            num_key_value_heads=hf.get("num_key_value_heads", n_heads),
            head_dim=hf.get("head_dim") or hf["hidden_size"] // n_heads,
            rms_norm_eps=hf.get("rms_norm_eps", 1e-5),
            rope_theta=float(hf.get("rope_theta", 10000.0)),
            rope_scaling=hf.get("rope_scaling"),
            max_position_embeddings=hf.get("max_position_embeddings", 131072),
            tie_word_embeddings=bool(hf.get("tie_word_embeddings", False)),
            attention_bias=bool(hf.get("attention_bias", mt == "qwen2")),
            qk_norm=mt in ("qwen3", "qwen3_moe", "gemma3_text"),
            num_experts=((hf.get("num_experts") or hf.get("num_local_experts") or 0) if mt.endswith("_moe")     # (newer HF configs: num_local_experts)
                         else (hf.get("n_routed_experts") or 0) if mt == "deepseek_v3"
                         else (hf.get("n_routed_experts") or 0) if (mt == "nemotron_h" and "moe" in hf["layers_block_type"]) else 0),
            num_experts_per_tok=hf.get("num_experts_per_tok", 0),
            moe_intermediate_size=hf.get("moe_intermediate_size", 0),
            norm_topk_prob=bool(hf.get("norm_topk_prob", True)),
            router_aux_loss_coef=float(hf.get("router_aux_loss_coef", 0.0)),
            bos_token_id=hf.get("bos_token_id"),
            eos_token_id=hf.get("eos_token_id"),
            pad_token_id=hf.get("pad_token_id"),
            torch_dtype=str(hf.get("torch_dtype") or hf.get("dtype") or "bfloat16").replace("torch.", ""),
            vision=hf.get("vision"),
            image_token_id=hf.get("image_token_id"),
        )
        if mt == "deepseek_v3":
            for k in ("kv_lora_rank", "q_lora_rank", "qk_nope_head_dim", "qk_rope_head_dim", "v_head_dim", "n_shared_experts",
                      "first_k_dense_replace", "n_group", "topk_group", "routed_scaling_factor"):
                if hf.get(k) is not None or k == "q_lora_rank":
                    setattr(cfg, k, hf.get(k))
            cfg.rope_interleave = bool(hf.get("rope_interleave", True))
            cfg.scoring_func = hf.get("scoring_func", "sigmoid")
            cfg.num_key_value_heads = cfg.num_attention_heads       # after decompression every head has its own keys and values
            cfg.head_dim = cfg.qk_nope_head_dim + cfg.qk_rope_head_dim   # what the attention kernels and the KV cache see (V is padded to it)
            rp = hf.get("rope_parameters") or hf.get("rope_scaling") or {}
            if isinstance(rp, dict) and rp.get("rope_type", rp.get("type", "default")) != "default":
                cfg.rope_scaling = {k: v for k, v in rp.items() if k != "rope_theta"}
                cfg.rope_theta = float(rp.get("rope_theta", cfg.rope_theta))
                m_all = float(rp.get("mscale_all_dim", 0) or 0)
                if m_all and float(rp["factor"]) > 1:      # the long-context recipe also sharpens the soft-max
                    ms = 0.1 * m_all * math.log(float(rp["factor"])) + 1.0
                    cfg.attn_scale = cfg.head_dim ** -0.5 * ms * ms
            elif isinstance(rp, dict) and rp.get("rope_theta"):
                cfg.rope_theta = float(rp["rope_theta"])
        if mt == "nemotron_h":
            cfg.layers_block_type = hf["layers_block_type"]
            cfg.use_rope, cfg.mlp_gated = False, False
            cfg.hidden_act = hf.get("mlp_hidden_act", "relu2")
            cfg.mlp_bias = bool(hf.get("mlp_bias", False))
            cfg.mamba_num_heads, cfg.mamba_head_dim = hf["mamba_num_heads"], hf["mamba_head_dim"]
            cfg.ssm_state_size = hf.get("ssm_state_size", 128)
            cfg.mamba_n_groups = hf.get("mamba_n_groups", hf.get("n_groups", 8))
            cfg.mamba_d_conv = hf.get("mamba_d_conv", hf.get("conv_kernel", 4))
            cfg.mamba_chunk_size = hf.get("mamba_chunk_size", hf.get("chunk_size", 128))
            cfg.mamba_conv_bias = bool(hf.get("mamba_conv_bias", hf.get("use_conv_bias", True)))
            cfg.mamba_proj_bias = bool(hf.get("mamba_proj_bias", hf.get("use_bias", False)))
            lim = hf.get("mamba_dt_limit", hf.get("time_step_limit"))
            cfg.mamba_dt_limit = [float(lim[0]), float(lim[1])] if lim is not None else None
            if cfg.is_moe:
                for k in ("n_shared_experts", "n_group", "topk_group", "routed_scaling_factor", "moe_latent_size"):
                    if hf.get(k) is not None:
                        setattr(cfg, k, hf[k])
                cfg.scoring_func = "sigmoid"
                cfg.moe_shared_expert_intermediate_size = hf.get("moe_shared_expert_intermediate_size", 0) or 0
        if mt == "gemma3_text":
            L = cfg.num_hidden_layers
            pattern = int(hf.get("sliding_window_pattern", 6) or 6)
            cfg.hidden_act = hf.get("hidden_activation", "gelu_pytorch_tanh")
            cfg.sandwich_norm, cfg.norm_offset = True, 1.0
            cfg.embed_scale = float(cfg.hidden_size) ** 0.5
            cfg.sliding_window = int(hf.get("sliding_window") or 0)
            cfg.layer_types = list(hf.get("layer_types") or ["sliding_attention" if (i + 1) % pattern else "full_attention" for i in range(L)])
            cfg.rope_local_theta = float(hf.get("rope_local_base_freq", 10000.0))
            cfg.attn_scale = float(hf.get("query_pre_attn_scalar", cfg.head_dim)) ** -0.5
            cfg.final_logit_softcap = float(hf.get("final_logit_softcapping") or 0.0)
            cfg.tie_word_embeddings = bool(hf.get("tie_word_embeddings", True))
            cfg.rms_norm_eps = hf.get("rms_norm_eps", 1e-6)
            rp = hf.get("rope_parameters")    # newer configs nest the RoPE settings per layer type
            if isinstance(rp, dict) and "full_attention" in rp:
                full, loc = rp["full_attention"], rp.get("sliding_attention", {})
                cfg.rope_theta = float(full.get("rope_theta", cfg.rope_theta))
                cfg.rope_scaling = {k: v for k, v in full.items() if k != "rope_theta"} if full.get("rope_type", "default") != "default" else None
                cfg.rope_local_theta = float(loc.get("rope_theta", cfg.rope_local_theta))
        for k, v in overrides.items():
            setattr(cfg, k, v)
        return cfg

    @classmethod
    def from_pretrained(cls, path: str, **overrides) -> "ModelConfig":
        with open(os.path.join(path, "config.json")) as f:
            return cls.from_hf_dict(json.load(f), **overrides)

    def save_pretrained(self, path: str) -> None:
        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, "config.json"), "w") as f:
            json.dump(self.to_hf_dict(), f, indent=2)


def rope_inv_freq(cfg: ModelConfig, device=None) -> torch.Tensor:
    """Inverse frequencies [head_dim/2] including the ``llama3`` / ``linear`` / ``yarn`` scaling rules."""
    D = cfg.qk_rope_head_dim if cfg.is_mla else cfg.head_dim     # MLA rotates only the decoupled rotary part of each head
    if not cfg.use_rope:   # a rotation by angle zero: the attention code paths stay the same
        z = torch.zeros(D // 2, dtype=torch.float32)
        return z.to(device) if device is not None else z
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    rs = cfg.rope_scaling or {}
    kind = rs.get("rope_type", rs.get("type", "default"))
    if kind == "linear":
        inv = inv / float(rs["factor"])
    elif kind == "llama3":
        factor, lo_f, hi_f = rs["factor"], rs.get("low_freq_factor", 1.0), rs.get("high_freq_factor", 4.0)
        old = rs.get("original_max_position_embeddings", 8192)
        wavelen = 2 * math.pi / inv
        smooth = ((old / wavelen) - lo_f) / (hi_f - lo_f)
        scaled = torch.where(wavelen > old / lo_f, inv / factor, inv)
        mid = (1 - smooth) * inv / factor + smooth * inv
        is_mid = (wavelen <= old / lo_f) & (wavelen >= old / hi_f)
        inv = torch.where(is_mid, mid, scaled)
    elif kind == "yarn":
        factor = float(rs["factor"])
        old = rs.get("original_max_position_embeddings", cfg.max_position_embeddings)
        beta_fast, beta_slow = rs.get("beta_fast", 32.0), rs.get("beta_slow", 1.0)

        def corr_dim(rot):
            return (D * math.log(old / (rot * 2 * math.pi))) / (2 * math.log(cfg.rope_theta))

        lo = max(math.floor(corr_dim(beta_fast)), 0)
        hi = min(math.ceil(corr_dim(beta_slow)), D // 2 - 1)
        ramp = ((torch.arange(D // 2, dtype=torch.float32) - lo) / max(hi - lo, 1e-3)).clamp(0, 1)
        inv = inv / factor * ramp + inv * (1 - ramp)
    return inv.to(device) if device is not None else inv


PRESETS: dict[str, dict] = {
    # Llama-3.1-8B: 32 layers, d 4096, GQA 32q/8kv, SwiGLU 14336, vocab 128256, RoPE theta 5e5 (llama3 scaling)
    "llama3.1-8b": dict(model_type="llama", vocab_size=128256, hidden_size=4096, intermediate_size=14336,
                        num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                        rms_norm_eps=1e-5, rope_theta=500000.0,
                        rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                          original_max_position_embeddings=8192),
                        bos_token_id=128000, eos_token_id=128001),
    "llama3.2-1b": dict(model_type="llama", vocab_size=128256, hidden_size=2048, intermediate_size=8192,
                        num_hidden_layers=16, num_attention_heads=32, num_key_value_heads=8, head_dim=64,
                        rms_norm_eps=1e-5, rope_theta=500000.0, tie_word_embeddings=True,
                        rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                          original_max_position_embeddings=8192)),
    "qwen3-32b": dict(model_type="qwen3", vocab_size=151936, hidden_size=5120, intermediate_size=25600,
                      num_hidden_layers=64, num_attention_heads=64, num_key_value_heads=8, head_dim=128,
                      rms_norm_eps=1e-6, rope_theta=1000000.0, qk_norm=True),
    "qwen3-30b-a3b": dict(model_type="qwen3_moe", vocab_size=151936, hidden_size=2048, intermediate_size=6144,
                          num_hidden_layers=48, num_attention_heads=32, num_key_value_heads=4, head_dim=128,
                          rms_norm_eps=1e-6, rope_theta=1000000.0, qk_norm=True, num_experts=128,
                          num_experts_per_tok=8, moe_intermediate_size=768, norm_topk_prob=True),
    "qwen2.5-0.5b": dict(model_type="qwen2", vocab_size=151936, hidden_size=896, intermediate_size=4864,
                         num_hidden_layers=24, num_attention_heads=14, num_key_value_heads=2, head_dim=64,
                         rms_norm_eps=1e-6, rope_theta=1000000.0, attention_bias=True, tie_word_embeddings=True),
    # the CPU/gloo oracle model: 4 layers, d 256, 4 heads, SwiGLU 688, vocab 2048
    # Gemma-3-1B (text): 26 layers, d 1152, 4 q / 1 kv heads of 256, GeGLU 6912, five sliding-window (512) layers per global one
    "gemma3-1b": dict(model_type="gemma3_text", vocab_size=262144, hidden_size=1152, intermediate_size=6912, num_hidden_layers=26,
                      num_attention_heads=4, num_key_value_heads=1, head_dim=256, rms_norm_eps=1e-6, rope_theta=1000000.0,
                      tie_word_embeddings=True, qk_norm=True, hidden_act="gelu_pytorch_tanh", sandwich_norm=True, embed_scale=1152 ** 0.5,
                      norm_offset=1.0, sliding_window=512, rope_local_theta=10000.0, attn_scale=256 ** -0.5,
                      layer_types=["full_attention" if (i + 1) % 6 == 0 else "sliding_attention" for i in range(26)]),
    "tiny-llama-oracle": dict(model_type="llama", vocab_size=2048, hidden_size=256, intermediate_size=688,
                              num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=4, head_dim=64,
                              rms_norm_eps=1e-5, rope_theta=10000.0),
    # tiny hybrid model for offline recipes and tests: Mamba-2, MLP, attention and expert blocks
    "tiny-nemotron-h": dict(model_type="nemotron_h", vocab_size=2048, hidden_size=256, intermediate_size=512, num_hidden_layers=6,
                            layers_block_type=["mamba", "mlp", "mamba", "attention", "mamba", "moe"], num_attention_heads=4,
                            num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-5, use_rope=False, mlp_gated=False, hidden_act="relu2",
                            mamba_num_heads=8, mamba_head_dim=64, ssm_state_size=32, mamba_n_groups=2, mamba_chunk_size=64,
                            num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128, n_shared_experts=1,
                            moe_shared_expert_intermediate_size=256, scoring_func="sigmoid"),
    # Nemotron-Nano-12B-v2-shaped (Mamba-2 / MLP blocks with six attention blocks; the reference's grpo-nano-v2-12b recipes)
    "nemotron-nano-12b-v2": dict(model_type="nemotron_h", vocab_size=131072, hidden_size=5120, intermediate_size=20480, num_hidden_layers=62,
                                 layers_block_type=[{"M": "mamba", "-": "mlp", "*": "attention"}[ch] for ch in
                                                    "M-M-M-M*-M-M-M-M*-M-M-M-M*-M-M-M-M*-M-M-M-M*-M-M-M-M*-M-M-M-M-"],
                                 num_attention_heads=40, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-5, use_rope=False,
                                 mlp_gated=False, hidden_act="relu2", mamba_num_heads=128, mamba_head_dim=80, ssm_state_size=128,
                                 mamba_n_groups=8, mamba_chunk_size=128),
    # Nemotron-3-Nano-30B-A3B-shaped (Mamba-2 / expert blocks with six attention blocks; the reference's grpo-nanov3 recipes)
    "nemotron-nano-30b-a3b-v3": dict(model_type="nemotron_h", vocab_size=131072, hidden_size=2688, intermediate_size=1856, num_hidden_layers=52,
                                     layers_block_type=[{"M": "mamba", "E": "moe", "*": "attention"}[ch] for ch in
                                                        "MEMEM*EMEMEM*EMEMEM*EMEMEM*EMEMEM*EMEMEMEM*EMEMEMEME"],
                                     num_attention_heads=32, num_key_value_heads=2, head_dim=128, rms_norm_eps=1e-5, use_rope=False,
                                     mlp_gated=False, hidden_act="relu2", mamba_num_heads=64, mamba_head_dim=64, ssm_state_size=128,
                                     mamba_n_groups=8, mamba_chunk_size=128, num_experts=128, num_experts_per_tok=6,
                                     moe_intermediate_size=1856, n_shared_experts=1, moe_shared_expert_intermediate_size=3712,
                                     scoring_func="sigmoid", routed_scaling_factor=2.5),
    # tiny vision-language model for offline recipes and tests: the oracle language model behind a 2-layer ViT
    "tiny-vlm": dict(model_type="llama", vocab_size=2048, hidden_size=256, intermediate_size=688,
                     num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=4, head_dim=64,
                     rms_norm_eps=1e-5, rope_theta=10000.0, image_token_id=511,
                     vision=dict(patch_size=4, channels=3, hidden_size=64, intermediate_size=128, num_layers=2, num_heads=4, max_patches=256)),
    # Qwen2-VL-7B-shaped: Qwen2-7B language model, 32-layer ViT of width 1280 on 14 x 14 patches
    "qwen2-vl-7b": dict(model_type="qwen2", vocab_size=152064, hidden_size=3584, intermediate_size=18944,
                        num_hidden_layers=28, num_attention_heads=28, num_key_value_heads=4, head_dim=128,
                        rms_norm_eps=1e-6, rope_theta=1000000.0, attention_bias=True, image_token_id=151655,
                        vision=dict(patch_size=14, channels=3, hidden_size=1280, intermediate_size=5120, num_layers=32, num_heads=16,
                                    max_patches=16384)),
}


def preset(name: str, **overrides) -> ModelConfig:
    cfg = ModelConfig(**PRESETS[name])
    for k, v in overrides.items():
        setattr(cfg, k, v)
    return cfg
