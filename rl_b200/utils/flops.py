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
