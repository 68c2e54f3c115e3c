"""FLOP accounting and MFU: per-architecture formulas plus a peak-throughput table.

The role of nemo_rl/utils/flops_tracker.py:43-129 and flops_formulas.py: model FLOPs per token for dense and
mixture-of-experts decoders (GEMMs + causal attention), and dense bf16 peaks per GPU used to turn achieved
throughput into model-FLOPs utilisation.
"""

from __future__ import annotations

import json
from pathlib import Path

# dense bf16 TFLOP/s per GPU (the halves of NVIDIA's with-sparsity figures)
PEAK_BF16_TFLOPS = {"B200": 2250.0, "GB200": 2450.0, "H100": 989.5, "H200": 989.5, "A100": 312.0}


def device_peak_tflops(name: str) -> float:
    for k, v in PEAK_BF16_TFLOPS.items():
        if k in name.upper():
            return v
    return float("nan")


def measured_peaks() -> dict:
    """Peaks measured on this machine pool, when the driver left them next to the package."""
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        return json.loads(p.read_text())
    return {}


def flops_per_token(cfg, seq_len: int) -> float:
    """Forward FLOPs per token at an average attended context of seq_len / 2 (causal)."""
    d, L = cfg.hidden_size, cfg.num_hidden_layers
    attn_proj = 2 * d * cfg.qkv_size + 2 * cfg.q_size * d
    attn_core = 2 * 2 * cfg.q_size * (seq_len / 2)  # QK^T and PV over the causal half
    if cfg.is_moe:
        ffn = 2 * 3 * d * cfg.moe_intermediate_size * cfg.num_experts_per_tok + 2 * d * cfg.num_experts
    else:
        ffn = 2 * 3 * d * cfg.intermediate_size
    head = 2 * d * (1 if getattr(cfg, "value_head", False) else cfg.vocab_size)
    return L * (attn_proj + attn_core + ffn) + head


def transformer_flops(cfg, tokens: int, seq_len: int, backward: bool = True) -> float:
    """Total FLOPs for ``tokens`` tokens; forward + backward counts 3x forward."""
    f = flops_per_token(cfg, seq_len) * tokens
    return 3.0 * f if backward else f


class FLOPTracker:
    def __init__(self, cfg, device_name: str = "B200"):
        self.cfg = cfg
        self.total = 0.0
        self.peak = device_peak_tflops(device_name)

    def track(self, tokens: int, seq_len: int, backward: bool = True) -> None:
        self.total += transformer_flops(self.cfg, tokens, seq_len, backward)

    def mfu(self, seconds: float, num_gpus: int) -> float:
        return self.total / seconds / num_gpus / (self.peak * 1e12) if seconds > 0 else 0.0

    def reset(self) -> None:
        self.total = 0.0


# ------------------------------------------------------------------------------------------------ per-architecture formulas
# Forward FLOPs of ONE sequence of ``seq`` tokens, built from components; ``hf`` is a HuggingFace-style config mapping
# (or any object with those attributes). A multiply-add counts 2. Causal attention counts half of the score / value
# products. Training = 3 x forward (backward re-does both GEMMs of every product). The families cover what the reference
# tabulates in nemo_rl/utils/flops_formulas.py (gpt3, llama, nemotron, mixtral, qwen2, qwen3 dense / MoE, deepseek-v3 with
# MLA, nemotron-h hybrids, bert): one formula per family there, one assembler of shared components here.
def _g(hf, key, default=None):
    if isinstance(hf, dict):
        return hf.get(key, default)
    return getattr(hf, key, default)


def attention_flops(seq: int, d: int, n_heads: int, n_kv_heads: int, head_dim: int, causal: bool = True) -> float:
    """q / k / v / o projections plus the score and value products of one layer."""
    q, kv = n_heads * head_dim, n_kv_heads * head_dim
    proj = 2 * seq * d * (q + 2 * kv) + 2 * seq * q * d
    core = 2 * 2 * seq * seq * q * (0.5 if causal else 1.0)
    return proj + core


def mla_attention_flops(seq: int, d: int, n_heads: int, q_lora: int, kv_lora: int, qk_nope: int, qk_rope: int, v_dim: int,
                        causal: bool = True) -> float:
    """Multi-head latent attention (DeepSeek-V2/V3): low-rank q and kv projections, decoupled rotary key."""
    qk = qk_nope + qk_rope
    q_proj = 2 * seq * (d * q_lora + q_lora * n_heads * qk) if q_lora else 2 * seq * d * n_heads * qk
    kv_proj = 2 * seq * (d * (kv_lora + qk_rope) + kv_lora * n_heads * (qk_nope + v_dim))
    o_proj = 2 * seq * n_heads * v_dim * d
    core = 2 * seq * seq * n_heads * (qk + v_dim) * (0.5 if causal else 1.0)
    return q_proj + kv_proj + o_proj + core


def mlp_flops(seq: int, d: int, ffn: int, gated: bool = True) -> float:
    return 2 * seq * d * ffn * (3 if gated else 2)


def moe_flops(seq: int, d: int, expert_ffn: int, top_k: int, n_experts: int, shared_ffn: int = 0, gated: bool = True) -> float:
    """Router + the ``top_k`` routed experts every token visits + shared experts."""
    return 2 * seq * d * n_experts + top_k * mlp_flops(seq, d, expert_ffn, gated) + (mlp_flops(seq, d, shared_ffn, gated) if shared_ffn else 0.0)


def mamba2_flops(seq: int, d: int, d_inner: int, d_state: int, n_groups: int, n_heads: int, conv_kernel: int = 4) -> float:
    """Mamba-2 mixer: input projection (z, x, B, C, dt), depthwise conv, selective scan, output projection."""
    in_proj = 2 * seq * d * (2 * d_inner + 2 * n_groups * d_state + n_heads)
    conv = 2 * seq * (d_inner + 2 * n_groups * d_state) * conv_kernel
    scan = 2 * 3 * seq * d_inner * d_state          # state update, decay, readout
    return in_proj + conv + scan + 2 * seq * d_inner * d


def head_flops(seq: int, d: int, vocab: int) -> float:
    return 2 * seq * d * vocab


def _dense_decoder(hf, seq: int, gated: bool = True) -> float:
    d, L = _g(hf, "hidden_size"), _g(hf, "num_hidden_layers")
    nh = _g(hf, "num_attention_heads")
    nkv = _g(hf, "num_key_value_heads") or nh
    hd = _g(hf, "head_dim") or d // nh
    layer = attention_flops(seq, d, nh, nkv, hd) + mlp_flops(seq, d, _g(hf, "intermediate_size"), gated)
    return L * layer + head_flops(seq, d, _g(hf, "vocab_size"))


def llama_flops(hf, seq: int) -> float:
    return _dense_decoder(hf, seq, gated=True)


qwen2_flops = mistral_flops = qwen3_flops = llama_flops


def gpt_flops(hf, seq: int) -> float:
    """GPT-2 / GPT-3 style: full multi-head attention and a non-gated 4d MLP."""
    return _dense_decoder(hf, seq, gated=False)


nemotron_flops = gpt_flops       # squared-ReLU MLP: two projections per layer, grouped-query attention


def moe_decoder_flops(hf, seq: int) -> float:
    """Mixtral / Qwen3-MoE: every layer is attention + routed experts (``decoder_sparse_step`` / ``mlp_only_layers`` select
    dense layers where a config has them)."""
    d, L = _g(hf, "hidden_size"), _g(hf, "num_hidden_layers")
    nh = _g(hf, "num_attention_heads")
    nkv = _g(hf, "num_key_value_heads") or nh
    hd = _g(hf, "head_dim") or d // nh
    n_exp = _g(hf, "num_experts") or _g(hf, "num_local_experts")
    top_k = _g(hf, "num_experts_per_tok")
    e_ffn = _g(hf, "moe_intermediate_size") or _g(hf, "intermediate_size")
    dense_layers = set(_g(hf, "mlp_only_layers") or [])
    step = _g(hf, "decoder_sparse_step") or 1
    total = 0.0
    for i in range(L):
        total += attention_flops(seq, d, nh, nkv, hd)
        if i in dense_layers or (i + 1) % step:
            total += mlp_flops(seq, d, _g(hf, "intermediate_size"))
        else:
            total += moe_flops(seq, d, e_ffn, top_k, n_exp, _g(hf, "shared_expert_intermediate_size") or 0)
    return total + head_flops(seq, d, _g(hf, "vocab_size"))


mixtral_flops = qwen3_moe_flops = moe_decoder_flops


def deepseek_v3_flops(hf, seq: int) -> float:
    """MLA attention in every layer; the first ``first_k_dense_replace`` layers have a dense MLP, the others routed + shared
    experts; multi-token-prediction modules add one more layer and head each."""
    d, L = _g(hf, "hidden_size"), _g(hf, "num_hidden_layers")
    attn = mla_attention_flops(seq, d, _g(hf, "num_attention_heads"), _g(hf, "q_lora_rank") or 0, _g(hf, "kv_lora_rank"),
                               _g(hf, "qk_nope_head_dim"), _g(hf, "qk_rope_head_dim"), _g(hf, "v_head_dim"))
    k_dense = _g(hf, "first_k_dense_replace") or 0
    shared = (_g(hf, "n_shared_experts") or 0) * _g(hf, "moe_intermediate_size")
    dense = mlp_flops(seq, d, _g(hf, "intermediate_size"))
    sparse = moe_flops(seq, d, _g(hf, "moe_intermediate_size"), _g(hf, "num_experts_per_tok"), _g(hf, "n_routed_experts"), shared)
    total = L * attn + k_dense * dense + (L - k_dense) * sparse + head_flops(seq, d, _g(hf, "vocab_size"))
    mtp = _g(hf, "num_nextn_predict_layers") or 0
    return total + mtp * (attn + sparse + head_flops(seq, d, _g(hf, "vocab_size")) + 2 * seq * 2 * d * d)


def nemotron_h_flops(hf, seq: int) -> float:
    """Hybrid Mamba-2 / attention / MLP stacks: ``hybrid_override_pattern`` has one letter per layer (M mamba, * attention,
    - MLP)."""
    d = _g(hf, "hidden_size")
    pattern = _g(hf, "hybrid_override_pattern") or ""
    nh = _g(hf, "num_attention_heads")
    nkv = _g(hf, "num_key_value_heads") or nh
    hd = _g(hf, "head_dim") or _g(hf, "attention_head_dim") or d // nh
    d_inner = (_g(hf, "mamba_num_heads") or 0) * (_g(hf, "mamba_head_dim") or 0) or 2 * d
    total = 0.0
    for ch in pattern:
        if ch == "M":
            total += mamba2_flops(seq, d, d_inner, _g(hf, "ssm_state_size") or 128, _g(hf, "n_groups") or 8,
                                  _g(hf, "mamba_num_heads") or d_inner // 64, _g(hf, "conv_kernel") or 4)
        elif ch == "*":
            total += attention_flops(seq, d, nh, nkv, hd)
        elif ch == "-":
            total += mlp_flops(seq, d, _g(hf, "intermediate_size"), gated=False)
    return total + head_flops(seq, d, _g(hf, "vocab_size"))


def bert_flops(hf, seq: int) -> float:
    d, L = _g(hf, "hidden_size"), _g(hf, "num_hidden_layers")
    nh = _g(hf, "num_attention_heads")
    layer = attention_flops(seq, d, nh, nh, d // nh, causal=False) + mlp_flops(seq, d, _g(hf, "intermediate_size"), gated=False)
    return L * layer + head_flops(seq, d, _g(hf, "vocab_size"))


def gemma3_flops(hf, seq: int) -> float:
    """Gemma 3: gated MLP everywhere; sliding-window layers attend to at most ``sliding_window`` keys per query, the
    global layers (every ``sliding_window_pattern``-th, or as listed in ``layer_types``) to the whole causal prefix."""
    d, L = _g(hf, "hidden_size"), _g(hf, "num_hidden_layers")
    nh = _g(hf, "num_attention_heads")
    nkv = _g(hf, "num_key_value_heads") or nh
    hd = _g(hf, "head_dim") or d // nh
    win = _g(hf, "sliding_window") or 0
    types = _g(hf, "layer_types")
    pattern = _g(hf, "sliding_window_pattern") or 6
    total = 0.0
    for i in range(L):
        sliding = (types[i] == "sliding_attention") if types else bool(win) and (i + 1) % pattern != 0
        a = attention_flops(seq, d, nh, nkv, hd)
        if sliding and win and seq > win:   # the core products see a band of width `win` instead of the causal triangle
            q = nh * hd
            a += 2 * 2 * seq * q * (win - (win * win) / (2.0 * seq)) - 2 * 2 * seq * seq * q * 0.5
        total += a + mlp_flops(seq, d, _g(hf, "intermediate_size"), True)
    return total + head_flops(seq, d, _g(hf, "vocab_size"))


FAMILY_FLOPS = {
    "llama": llama_flops, "mistral": mistral_flops, "qwen2": qwen2_flops, "qwen3": qwen3_flops, "gemma3": gemma3_flops,
    "gemma3_text": gemma3_flops,
    "gpt2": gpt_flops, "gpt3": gpt_flops, "nemotron": nemotron_flops, "mixtral": mixtral_flops, "qwen3_moe": qwen3_moe_flops,
    "qwen2_moe": moe_decoder_flops, "deepseek_v3": deepseek_v3_flops, "deepseek_v2": deepseek_v3_flops, "nemotron_h": nemotron_h_flops,
    "bert": bert_flops,
}


def model_flops(hf, seq: int, batch: int = 1, backward: bool = True, model_type: str = "") -> float:
    """FLOPs of ``batch`` sequences of ``seq`` tokens for the architecture named by ``model_type`` (default: the config's
    own ``model_type``); unknown families fall back to the dense decoder formula."""
    fam = FAMILY_FLOPS.get(model_type or _g(hf, "model_type") or "llama", llama_flops)
    f = fam(hf, seq) * batch
    return 3.0 * f if backward else f
