"""Quantisation-aware RL: the policy trains, scores and generates through quantise-dequantise ("fake quant") operators on
chosen linear layers, so the distribution it is optimised for is the one its quantised deployment will have.

``policy.quant_cfg`` names a recipe: a built-in (``NVFP4_DEFAULT_CFG``: block-16 NVFP4 weights and inputs of every linear
layer but the output head and the routers; ``NVFP4_W4A16`` / ``nvfp4_a16``: weights only; ``NVFP4_EXPERTS``: routed experts
only; ``FP8_DEFAULT_CFG``: per-tensor E4M3) or a YAML file in the ModelOpt PTQ layout (``quantize.quant_cfg``: an ORDERED list
of ``{quantizer_name: wildcard, enable: bool, cfg: {num_bits, block_sizes}}``; later entries win) matched against
``<HF module name>.weight_quantizer`` / ``.input_quantizer``. Calibration (``algorithm: max``) runs a few forward passes and
freezes each input quantizer's tensor-level range; weight ranges follow the weights.

How it reaches the math: :func:`attach` hangs a :class:`Quantizers` object on every chosen parameter; ``ops.functional.linear``
and the expert MLP consult it. Under ``no_grad`` (log-prob passes, the generation engine) the quantised weights are cached until
:func:`QatState.weights_changed`. :func:`export_quantized` writes the real 4-bit tensors (packed values, E4M3 block scales,
fp32 tensor scales, input scales) with ``hf_quant_config.json`` for NVFP4 serving stacks.

Role of nemo_rl/modelopt/utils.py (recipe resolution, ignore patterns), modelopt/models/policy/workers/utils.py (``quantize_model``
with its calibration loop) and examples/modelopt/export_quantized_to_hf.py.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from fnmatch import fnmatchcase
from typing import Any, Iterable, Optional

import torch

from rl_b200.ops.nvfp4 import fake_quant, quantize_nvfp4

_NV = dict(num_bits="e2m1", block_sizes={-1: 16, "type": "dynamic", "scale_bits": "e4m3"})
_F8 = dict(num_bits="e4m3")
_OFF_DEFAULT = [dict(quantizer_name=p, enable=False) for p in ("*lm_head*", "*output_layer*", "*router*", "*mlp.gate.*", "*mixer.gate.*",
                                                               "*block_sparse_moe.gate*")]
BUILTIN_RECIPES: dict[str, dict] = {
    "NVFP4_DEFAULT_CFG": dict(algorithm="max", quant_cfg=[dict(quantizer_name="*weight_quantizer", enable=True, cfg=_NV),
                                                          dict(quantizer_name="*input_quantizer", enable=True, cfg=_NV)] + _OFF_DEFAULT),
    "NVFP4_W4A16": dict(algorithm="max", quant_cfg=[dict(quantizer_name="*weight_quantizer", enable=True, cfg=_NV),
                                                    dict(quantizer_name="*input_quantizer", enable=False)] + _OFF_DEFAULT),
    "NVFP4_EXPERTS": dict(algorithm="max", quant_cfg=[dict(quantizer_name="*", enable=False),
                                                      dict(quantizer_name="*.experts.*weight_quantizer", enable=True, cfg=_NV),
                                                      dict(quantizer_name="*.experts.*input_quantizer", enable=True, cfg=_NV)]),
    "FP8_DEFAULT_CFG": dict(algorithm="max", quant_cfg=[dict(quantizer_name="*weight_quantizer", enable=True, cfg=_F8),
                                                        dict(quantizer_name="*input_quantizer", enable=True, cfg=_F8)] + _OFF_DEFAULT),
}
BUILTIN_RECIPES["nvfp4_a16"] = BUILTIN_RECIPES["NVFP4_W4A16"]


class QatState:
    """Process-wide switch and weight version (cached quantised weights are rebuilt when the version moves)."""

    enabled = True
    version = 0

    @classmethod
    def weights_changed(cls) -> None:
        cls.version += 1


def resolve_quant_cfg(quant_cfg: str) -> dict:
    """Built-in name or YAML path -> ``{"algorithm": ..., "quant_cfg": [entries]}``."""
    if quant_cfg in BUILTIN_RECIPES:
        return BUILTIN_RECIPES[quant_cfg]
    if os.path.exists(quant_cfg):
        import yaml

        with open(quant_cfg) as f:
            doc = yaml.safe_load(f)
        doc = doc.get("quantize", doc) if isinstance(doc, dict) else None
        if not isinstance(doc, dict) or "quant_cfg" not in doc:
            raise ValueError(f"quantisation recipe '{quant_cfg}' needs a 'quant_cfg' list (optionally under 'quantize:')")
        return {"algorithm": doc.get("algorithm", "max"), "quant_cfg": list(doc["quant_cfg"])}
    raise ValueError(f"unknown quant_cfg '{quant_cfg}': a built-in name ({', '.join(sorted(BUILTIN_RECIPES))}) or the path of a YAML recipe")


def _kind_of(cfg: Optional[dict]) -> str:
    nb = (cfg or {}).get("num_bits", "e2m1")
    if nb in ("e2m1", (2, 1), [2, 1]):
        bs = (cfg or {}).get("block_sizes") or {}
        blk = bs.get(-1, bs.get("-1", 16))
        if int(blk) != 16 or bs.get("scale_bits", "e4m3") not in ("e4m3", (4, 3), [4, 3]):
            raise ValueError("NVFP4 quantizers use blocks of 16 with E4M3 scales")
        return "nvfp4"
    if nb in ("e4m3", (4, 3), [4, 3], 8):
        return "fp8"
    raise ValueError(f"unsupported quantizer format num_bits={nb!r}")


def quantizer_setting(entries: Iterable[dict], name: str) -> Optional[str]:
    """The format ("nvfp4" / "fp8") the ordered recipe leaves enabled for quantizer ``name``, or None."""
    out = None
    for e in entries:
        if fnmatchcase(name, e["quantizer_name"]):
            out = _kind_of(e.get("cfg")) if e.get("enable", True) else None
    return out


@dataclass
class Quantizers:
    """What ``linear`` applies for one parameter. ``pieces``: row ranges holding separate checkpoint tensors (q / k / v,
    gate / up), each with its own tensor-level scale as in a real export."""

    name: str
    weight: Optional[str] = None
    input: Optional[str] = None
    pieces: list = field(default_factory=list)
    input_amax: Optional[torch.Tensor] = None      # frozen by calibration; None: the running batch's own maximum
    calibrating: bool = False
    _seen: Optional[torch.Tensor] = None
    _cache: Any = None

    def q_weight(self, w: torch.Tensor) -> torch.Tensor:
        if self.weight is None:
            return w
        grad = w.requires_grad and torch.is_grad_enabled()
        if not grad and self._cache is not None and self._cache[0] == QatState.version and self._cache[1].shape == w.shape:
            return self._cache[1]
        if w.shape[-1] % 16 and self.weight == "nvfp4":
            raise ValueError(f"{self.name}: NVFP4 needs an input width that is a multiple of 16")
        rows = self.pieces or [(0, w.shape[-2])]

        def one(t):   # stacked experts: every expert's matrix is a checkpoint tensor of its own, with its own tensor-level scale
            return fake_quant(t, self.weight, t.detach().abs().amax(dim=(-2, -1), keepdim=True) if t.dim() == 3 else None, clip=False)

        out = torch.cat([one(w[..., a:b, :]) for a, b in rows], dim=-2) if len(rows) > 1 else one(w)
        if not grad:
            self._cache = (QatState.version, out.detach())
        return out

    def q_input(self, x: torch.Tensor) -> torch.Tensor:
        if self.input is None or x.numel() == 0:
            return x
        if self.calibrating:
            m = x.detach().abs().amax().float()
            self._seen = m if self._seen is None else torch.maximum(self._seen, m)
            return x
        return fake_quant(x, self.input, self.input_amax)

    def finish_calibration(self, group=None) -> None:
        self.calibrating = False
        if self._seen is not None:
            if group is not None and torch.distributed.is_initialized():
                torch.distributed.all_reduce(self._seen, op=torch.distributed.ReduceOp.MAX, group=group)
            self.input_amax = self._seen.clone()
        self._seen = None


def attach(model, recipe: dict) -> dict[str, Quantizers]:
    """Decides, parameter by parameter, what the recipe enables and hangs the quantizers on the parameters."""
    from rl_b200.models.hf_io import _model_map

    entries = recipe["quant_cfg"]
    params = dict(model.named_parameters())
    by_param: dict[str, list] = {}
    for hf, loc, rows, e, hs in _model_map(model):
        if hf.endswith(".weight") and loc in params and params[loc].dim() >= 2 and "norm" not in hf and "embed" not in hf and "conv1d" not in hf:
            by_param.setdefault(loc, []).append((hf[: -len(".weight")], rows, e))
    out = {}
    for loc, items in by_param.items():
        p = params[loc]
        mods = sorted({m for m, _, _ in items})
        wk = {quantizer_setting(entries, m + ".weight_quantizer") for m in mods}
        ik = {quantizer_setting(entries, m + ".input_quantizer") for m in mods}
        if len(wk) > 1 or len(ik) > 1:
            raise ValueError(f"{loc}: the recipe treats the tensors fused into this parameter differently ({mods[:3]}...)")
        w_kind, i_kind = wk.pop(), ik.pop()
        if w_kind is None and i_kind is None:
            continue
        pieces = sorted({rows for _, rows, e in items if rows is not None})
        q = Quantizers(loc, w_kind, i_kind, pieces=list(pieces))
        p._rlb_qat = q
        out[loc] = q
    return out


def detach(model) -> None:
    for p in model.parameters():
        if hasattr(p, "_rlb_qat"):
            del p._rlb_qat


@torch.no_grad()
def calibrate(quantizers: dict[str, Quantizers], forward_batches, group=None) -> int:
    """``algorithm: max``: runs ``forward_batches`` (an iterable of zero-argument callables, each one forward pass) with the input
    quantizers observing, then freezes their ranges (maximum over the data-parallel group). Returns the passes run."""
    for q in quantizers.values():
        q.calibrating = q.input is not None
    n = 0
    try:
        for run in forward_batches:
            run()
            n += 1
    finally:
        for q in quantizers.values():
            if q.input is not None:
                q.finish_calibration(group)
    return n


def state_dict(quantizers: dict[str, Quantizers]) -> dict:
    return {n: q.input_amax.detach().cpu() for n, q in quantizers.items() if q.input_amax is not None}


def load_state_dict(quantizers: dict[str, Quantizers], sd: dict) -> None:
    for n, t in sd.items():
        if n in quantizers:
            p = quantizers[n]
            p.input_amax = t.to(p.input_amax.device if p.input_amax is not None else "cpu").float()


@torch.no_grad()
def export_quantized(model, quantizers: dict[str, Quantizers], path: str) -> dict:
    """Writes the deployment form: for every NVFP4-quantised checkpoint tensor ``<name>.weight`` (packed uint8, two values per
    byte), ``.weight_scale`` (E4M3 per block of 16), ``.weight_scale_2`` (fp32 per tensor) and, with input quantisation,
    ``.input_scale``; everything else as it is; ``hf_quant_config.json`` names the algorithm and the modules left alone."""
    from safetensors.torch import save_file

    from rl_b200.models.hf_io import _model_map, iter_hf_shards

    os.makedirs(path, exist_ok=True)
    out, excluded, algo = {}, [], None
    where = {hf: loc for hf, loc, rows, e, hs in _model_map(model)}
    for hf, t, hs in iter_hf_shards(model):
        q = quantizers.get(where.get(hf, ""))
        if q is None or q.weight != "nvfp4" or not hf.endswith(".weight"):
            out[hf] = t.detach().contiguous().cpu()
            if hf.endswith(".weight") and t.dim() >= 2 and "norm" not in hf and "embed" not in hf:
                excluded.append(hf[: -len(".weight")])
            continue
        packed, sb, s2 = quantize_nvfp4(t.detach())
        base = hf[: -len(".weight")]
        out[hf], out[base + ".weight_scale"], out[base + ".weight_scale_2"] = packed.cpu(), sb.cpu(), s2.cpu()
        if q.input == "nvfp4":
            a = q.input_amax if q.input_amax is not None else torch.tensor(0.0)
            out[base + ".input_scale"] = (a.float() / (6.0 * 448.0)).reshape(()).cpu()
        algo = "NVFP4" if (q.input == "nvfp4" or algo == "NVFP4") else (algo or "W4A16_NVFP4")
    save_file(out, os.path.join(path, "model.safetensors"))
    meta = {"producer": {"name": "rl_b200"}, "quantization": {"quant_algo": algo, "group_size": 16, "exclude_modules": sorted(set(excluded))}}
    with open(os.path.join(path, "hf_quant_config.json"), "w") as f:
        json.dump(meta, f, indent=2)
    model.cfg.save_pretrained(path)
    return meta
