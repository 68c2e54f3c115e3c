"""HuggingFace checkpoint interchange: safetensors in HF tensor names <-> this package's fused parameters.

The on-disk contract is the HF layout (``config.json`` + ``model-0000x-of-0000y.safetensors`` +
``model.safetensors.index.json``) with per-projection names (``q_proj``, ``k_proj``, ``v_proj``, ``gate_proj``,
``up_proj``...). In memory q/k/v and gate/up are fused, and MoE experts are stacked; this module is the single place
that knows both namings. The same mapping names the logical tensors of a weight refit
(nemo_rl/models/policy/workers/dtensor_policy_worker_v2.py:1074 ships HF names as the wire format).
"""

from __future__ import annotations

import json
import os
import re
from typing import Callable, Iterator, Optional

import torch

from .config import ModelConfig
from .transformer import CausalLM


def hf_name_map(cfg: ModelConfig, tp_rank: int = 0, tp_size: int = 1, layer_offset: int = 0, num_local_layers: Optional[int] = None,
                first_stage: bool = True, last_stage: bool = True, layer_ids=None):
    """Rows of (hf_name, local_name, local_rows or None, expert index or None, hf_slice or None).

    The HF tensor, restricted to ``hf_slice = (dim, start, length)`` when this rank holds a tensor-parallel shard of it,
    is rows ``local_rows`` of the local parameter (of global expert ``e`` when the local parameter is expert-stacked).
    Local layer ``j`` is HF layer ``layer_offset + j`` (pipeline stages own contiguous layer ranges), or ``layer_ids[j]`` when
    the stage interleaves several runs of layers."""
    n_layers = cfg.num_hidden_layers - layer_offset if num_local_layers is None else num_local_layers
    ids = list(layer_ids) if layer_ids is not None else [layer_offset + j for j in range(n_layers)]
    n_layers = len(ids)
    tied = cfg.tie_word_embeddings and not cfg.value_head
    rows = []
    hybrid = cfg.is_hybrid     # Nemotron-H names: model.embeddings, model.norm_f, layers.N.norm + layers.N.mixer.*
    if first_stage or (last_stage and tied):
        rows.append(("model.embeddings.weight" if hybrid else "model.embed_tokens.weight", "embed_tokens", None, None, None))
    if last_stage:
        rows.append(("model.norm_f.weight" if hybrid else "model.norm.weight", "norm", None, None, None))
        if cfg.value_head:
            rows.append(("score.weight", "score", (0, 1), None, None))
        elif not tied:
            vl = cfg.vocab_size // tp_size
            rows.append(("lm_head.weight", "lm_head", None, None, (0, tp_rank * vl, vl) if tp_size > 1 else None))
    # (Gemma's two extra norms per layer are added with the other layer tensors below)
    if cfg.vision is not None and first_stage:   # vision tower: replicated, stored under its own names
        from .vision import vision_config

        nv = vision_config(cfg)["num_layers"]
        leaves = ["patch_embed", "pos_embed", "merger_norm", "merger_fc1", "merger_fc2"]
        leaves += [f"blocks.{i}.{k}" for i in range(nv) for k in ("attn_norm", "qkv", "proj", "mlp_norm", "fc1", "fc2")]
        rows += [(f"visual.{k}.weight", f"visual.{k}", None, None, None) for k in leaves]
    q, kv = cfg.q_size // tp_size, cfg.kv_size // tp_size

    def sl(dim, n):  # this rank's slice of a dimension of (global) length n * tp_size
        return (dim, tp_rank * n, n) if tp_size > 1 else None

    for j in range(n_layers if hybrid else 0):
        hp, lp = f"model.layers.{ids[j]}", f"layers.{j}"
        mx, kind = f"{hp}.mixer", cfg.block_type(ids[j])
        rows.append((f"{hp}.norm.weight", f"{lp}.norm", None, None, None))
        if kind == "mamba":
            rows += [(f"{mx}.in_proj.weight", f"{lp}.mamba.in_proj", None, None, None),
                     (f"{mx}.conv1d.weight", f"{lp}.mamba.conv_weight", None, None, None),
                     (f"{mx}.dt_bias", f"{lp}.mamba.dt_bias", None, None, None),
                     (f"{mx}.A_log", f"{lp}.mamba.A_log", None, None, None),
                     (f"{mx}.D", f"{lp}.mamba.D", None, None, None),
                     (f"{mx}.norm.weight", f"{lp}.mamba.norm", None, None, None),
                     (f"{mx}.out_proj.weight", f"{lp}.mamba.out_proj", None, None, None)]
            if cfg.mamba_conv_bias:
                rows.append((f"{mx}.conv1d.bias", f"{lp}.mamba.conv_bias", None, None, None))
            if cfg.mamba_proj_bias:
                rows += [(f"{mx}.in_proj.bias", f"{lp}.mamba.in_proj_bias", None, None, None),
                         (f"{mx}.out_proj.bias", f"{lp}.mamba.out_proj_bias", None, None, None)]
        elif kind == "attention":   # replicated over a tensor-parallel group
            qf, kvf = cfg.q_size, cfg.kv_size
            rows += [(f"{mx}.q_proj.weight", f"{lp}.self_attn.qkv_proj", (0, qf), None, None),
                     (f"{mx}.k_proj.weight", f"{lp}.self_attn.qkv_proj", (qf, qf + kvf), None, None),
                     (f"{mx}.v_proj.weight", f"{lp}.self_attn.qkv_proj", (qf + kvf, qf + 2 * kvf), None, None),
                     (f"{mx}.o_proj.weight", f"{lp}.self_attn.o_proj", None, None, None)]
        elif kind == "mlp":
            f = cfg.intermediate_size // tp_size
            rows += [(f"{mx}.up_proj.weight", f"{lp}.mlp.up_proj", None, None, sl(0, f)),
                     (f"{mx}.down_proj.weight", f"{lp}.mlp.down_proj", None, None, sl(1, f))]
        else:
            rows += [(f"{mx}.gate.weight", f"{lp}.mlp.router", None, None, None),
                     (f"{mx}.gate.e_score_correction_bias", f"{lp}.mlp.e_score_correction_bias", None, None, None)]
            if cfg.moe_latent_size:
                rows += [(f"{mx}.fc1_latent_proj.weight", f"{lp}.mlp.fc1_latent_proj", None, None, None),
                         (f"{mx}.fc2_latent_proj.weight", f"{lp}.mlp.fc2_latent_proj", None, None, None)]
            if cfg.n_shared_experts:
                rows += [(f"{mx}.shared_experts.up_proj.weight", f"{lp}.mlp.shared_experts.up_proj", None, None, None),
                         (f"{mx}.shared_experts.down_proj.weight", f"{lp}.mlp.shared_experts.down_proj", None, None, None)]
            for e in range(cfg.num_experts):
                rows += [(f"{mx}.experts.{e}.up_proj.weight", f"{lp}.mlp.up_proj", None, e, None),
                         (f"{mx}.experts.{e}.down_proj.weight", f"{lp}.mlp.down_proj", None, e, None)]
    for j in range(0 if hybrid else n_layers):
        hp, lp = f"model.layers.{ids[j]}", f"layers.{j}"
        rows += [
            (f"{hp}.input_layernorm.weight", f"{lp}.input_layernorm", None, None, None),
            (f"{hp}.post_attention_layernorm.weight", f"{lp}.post_attention_layernorm", None, None, None),
        ]
        if cfg.is_mla:   # latent attention (not tensor parallel): its projections keep their own names
            sa = f"{hp}.self_attn"
            if cfg.q_lora_rank:
                rows += [(f"{sa}.q_a_proj.weight", f"{lp}.self_attn.q_a_proj", None, None, None),
                         (f"{sa}.q_a_layernorm.weight", f"{lp}.self_attn.q_a_layernorm", None, None, None),
                         (f"{sa}.q_b_proj.weight", f"{lp}.self_attn.q_b_proj", None, None, None)]
            else:
                rows.append((f"{sa}.q_proj.weight", f"{lp}.self_attn.q_proj", None, None, None))
            rows += [(f"{sa}.kv_a_proj_with_mqa.weight", f"{lp}.self_attn.kv_a_proj", None, None, None),
                     (f"{sa}.kv_a_layernorm.weight", f"{lp}.self_attn.kv_a_layernorm", None, None, None),
                     (f"{sa}.kv_b_proj.weight", f"{lp}.self_attn.kv_b_proj", None, None, None),
                     (f"{sa}.o_proj.weight", f"{lp}.self_attn.o_proj", None, None, None)]
        else:
            rows += [
                (f"{hp}.self_attn.q_proj.weight", f"{lp}.self_attn.qkv_proj", (0, q), None, sl(0, q)),
                (f"{hp}.self_attn.k_proj.weight", f"{lp}.self_attn.qkv_proj", (q, q + kv), None, sl(0, kv)),
                (f"{hp}.self_attn.v_proj.weight", f"{lp}.self_attn.qkv_proj", (q + kv, q + 2 * kv), None, sl(0, kv)),
                (f"{hp}.self_attn.o_proj.weight", f"{lp}.self_attn.o_proj", None, None, sl(1, q)),
            ]
        if cfg.attention_bias:
            rows += [
                (f"{hp}.self_attn.q_proj.bias", f"{lp}.self_attn.qkv_bias", (0, q), None, sl(0, q)),
                (f"{hp}.self_attn.k_proj.bias", f"{lp}.self_attn.qkv_bias", (q, q + kv), None, sl(0, kv)),
                (f"{hp}.self_attn.v_proj.bias", f"{lp}.self_attn.qkv_bias", (q + kv, q + 2 * kv), None, sl(0, kv)),
            ]
        if cfg.qk_norm and not cfg.is_mla:
            rows += [(f"{hp}.self_attn.q_norm.weight", f"{lp}.self_attn.q_norm", None, None, None),
                     (f"{hp}.self_attn.k_norm.weight", f"{lp}.self_attn.k_norm", None, None, None)]
        if cfg.sandwich_norm:
            rows += [(f"{hp}.pre_feedforward_layernorm.weight", f"{lp}.pre_feedforward_layernorm", None, None, None),
                     (f"{hp}.post_feedforward_layernorm.weight", f"{lp}.post_feedforward_layernorm", None, None, None)]
        if cfg.layer_is_moe(ids[j]):
            f = cfg.moe_intermediate_size
            rows.append((f"{hp}.mlp.gate.weight", f"{lp}.mlp.router", None, None, None))
            if cfg.scoring_func == "sigmoid":
                rows.append((f"{hp}.mlp.gate.e_score_correction_bias", f"{lp}.mlp.e_score_correction_bias", None, None, None))
            if cfg.n_shared_experts:
                fs = f * cfg.n_shared_experts
                rows += [(f"{hp}.mlp.shared_experts.gate_proj.weight", f"{lp}.mlp.shared_experts.gate_up_proj", (0, fs), None, None),
                         (f"{hp}.mlp.shared_experts.up_proj.weight", f"{lp}.mlp.shared_experts.gate_up_proj", (fs, 2 * fs), None, None),
                         (f"{hp}.mlp.shared_experts.down_proj.weight", f"{lp}.mlp.shared_experts.down_proj", None, None, None)]
            for e in range(cfg.num_experts):
                rows += [
                    (f"{hp}.mlp.experts.{e}.gate_proj.weight", f"{lp}.mlp.gate_up_proj", (0, f), e, None),
                    (f"{hp}.mlp.experts.{e}.up_proj.weight", f"{lp}.mlp.gate_up_proj", (f, 2 * f), e, None),
                    (f"{hp}.mlp.experts.{e}.down_proj.weight", f"{lp}.mlp.down_proj", None, e, None),
                ]
        else:
            f = cfg.intermediate_size // tp_size
            rows += [
                (f"{hp}.mlp.gate_proj.weight", f"{lp}.mlp.gate_up_proj", (0, f), None, sl(0, f)),
                (f"{hp}.mlp.up_proj.weight", f"{lp}.mlp.gate_up_proj", (f, 2 * f), None, sl(0, f)),
                (f"{hp}.mlp.down_proj.weight", f"{lp}.mlp.down_proj", None, None, sl(1, f)),
            ]
    return rows


def _local(model: CausalLM) -> dict[str, torch.Tensor]:
    out = dict(model.named_parameters())
    if hasattr(model, "named_buffers"):   # (views that stand in for a model, e.g. its gradients, have parameters only)
        out.update({n: b for n, b in model.named_buffers() if n.endswith("e_score_correction_bias")})   # stored in checkpoints, not trained
    return out


def _model_map(model: CausalLM):
    return hf_name_map(model.cfg, model.tp.rank, model.tp.world, model.layer_offset, len(model.layers), model.first_stage, model.last_stage,
                       layer_ids=getattr(model, "layer_ids", None))


def iter_hf_shards(model: CausalLM) -> Iterator[tuple[str, torch.Tensor, Optional[tuple[int, int, int]]]]:
    """Yields (hf_name, local tensor view, hf_slice) for every logical HF tensor (or shard of one) this rank holds."""
    cfg = model.cfg
    params = _local(model)
    ep_rank, ep_size = (model.ep.rank, model.ep.world) if model.ep is not None else (0, 1)
    per = cfg.num_experts // ep_size if cfg.is_moe else 0
    for hf, loc, rows, e, hs in _model_map(model):
        p = params[loc]
        if e is not None:
            if not (ep_rank * per <= e < (ep_rank + 1) * per):
                continue
            p = p[e - ep_rank * per]
        yield hf, (p if rows is None else p[rows[0] : rows[1]]), hs


def hf_full_shape(local_shape: tuple, hf_slice, tp_size: int) -> tuple:
    """Shape of the whole HF tensor given the shape of this rank's slice of it."""
    if hf_slice is None:
        return tuple(local_shape)
    full = list(local_shape)
    full[hf_slice[0]] *= tp_size
    return tuple(full)


def iter_hf_tensors(model: CausalLM) -> Iterator[tuple[str, torch.Tensor]]:
    """Yields (hf_name, FULL tensor). Without model parallelism these are views of the parameters; with tensor
    parallelism every shard is all-gathered over the tp group (collective: all tp ranks must iterate together)."""
    from rl_b200.parallel.tensor import all_gather_rows

    tp = model.tp
    off = float(getattr(model.cfg, "norm_offset", 0.0) or 0.0)
    for hf, t, hs in iter_hf_shards(model):
        if off and _is_norm_weight(hf):
            yield hf, (t.detach().float() - off).to(t.dtype)    # checkpoints of this family store w - offset
        elif hs is None or tp.world == 1:
            yield hf, t
        elif hs[0] == 0:
            yield hf, all_gather_rows(t.detach(), tp.group, tp.world)
        else:
            yield hf, all_gather_rows(t.detach().t().contiguous(), tp.group, tp.world).t().contiguous()


def _is_norm_weight(hf_name: str) -> bool:
    return hf_name.endswith("norm.weight") or hf_name.endswith("layernorm.weight")


@torch.no_grad()
def load_hf_tensors(model: CausalLM, get: Callable[[str], Optional[torch.Tensor]], strict: bool = True) -> list[str]:
    """Copies HF-named tensors (as returned by ``get(name)``) into the fused (and possibly sharded) parameters.
    Returns missing names. Families whose checkpoints store RMSNorm weights as ``w - 1`` (Gemma) get the offset added
    here and removed by :func:`iter_hf_tensors`, so the buffers always hold the multiplier itself."""
    missing = []
    off = float(getattr(model.cfg, "norm_offset", 0.0) or 0.0)
    for hf, dst, hs in iter_hf_shards(model):
        src = get(hf)
        if src is None:
            missing.append(hf)
            continue
        if hs is not None:
            src = src.narrow(hs[0], hs[1], hs[2])
        if tuple(src.shape) != tuple(dst.shape):
            raise ValueError(f"{hf}: checkpoint shape {tuple(src.shape)} != model shape {tuple(dst.shape)}")
        if off and _is_norm_weight(hf):
            src = src.float() + off
        dst.copy_(src.to(dst.dtype))
    if strict and missing:
        raise KeyError(f"{len(missing)} tensors missing from checkpoint, first: {missing[:5]}")
    return missing


def save_roles(state=None) -> tuple[bool, bool, str]:
    """(takes part in the save, writes dense tensors, file-name suffix) for this rank under the current parallel layout.

    Tensor-parallel ranks of the writing replica all take part (shards are all-gathered) and rank 0 of the group writes;
    every pipeline stage writes its own layers; every rank of the first expert-parallel group writes its own experts."""
    from rl_b200.parallel.state import get_state

    st = state or get_state()
    if st.world == 1:
        return True, True, ""
    plane = st.dp_rank * st.cp + st.cp_rank
    takes_part = plane < max(1, st.ep)
    writes_dense = plane == 0
    suffix = "" if st.pp * st.ep == 1 else f"-pp{st.pp_rank}-ep{st.ep_rank}"
    return takes_part, writes_dense, suffix


def save_pretrained(model: CausalLM, path: str, max_shard_bytes: int = 5 * 1024**3, dtype: Optional[torch.dtype] = None) -> None:
    """Writes an HF-layout checkpoint (config + sharded safetensors + index). Under model parallelism this is a
    collective over the tensor-parallel group; pipeline stages and expert-parallel ranks write separate shard files."""
    from safetensors.torch import save_file

    takes_part, writes_dense, suffix = save_roles()
    if not takes_part:
        return
    os.makedirs(path, exist_ok=True)
    is_writer = model.tp.rank == 0
    if is_writer and writes_dense and model.first_stage:
        model.cfg.save_pretrained(path)
    shards: list[dict[str, torch.Tensor]] = [{}]
    size = 0
    for name, t in iter_hf_tensors(model):  # collective over the tp group when the model is tensor parallel
        if not is_writer or not (writes_dense or ".mlp.experts." in name):
            continue
        if name == "model.embed_tokens.weight" and not model.first_stage:
            continue  # the last stage's copy of a tied table
        t = t.detach().to("cpu", dtype or t.dtype).contiguous()
        nbytes = t.numel() * t.element_size()
        if size + nbytes > max_shard_bytes and shards[-1]:
            shards.append({})
            size = 0
        shards[-1][name] = t
        size += nbytes
    if not is_writer:
        return
    n = len(shards)
    weight_map, total = {}, 0
    for i, sh in enumerate(shards):
        if not sh:
            continue
        fname = f"model{suffix}.safetensors" if n == 1 else f"model{suffix}-{i + 1:05d}-of-{n:05d}.safetensors"
        save_file(sh, os.path.join(path, fname), metadata={"format": "pt"})
        for k, t in sh.items():
            weight_map[k] = fname
            total += t.numel() * t.element_size()
    if n > 1 and not suffix:
        with open(os.path.join(path, "model.safetensors.index.json"), "w") as f:
            json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f, indent=2)


class _SafetensorsDir:
    """Lazy reader over an HF checkpoint directory (single file or sharded with an index)."""

    def __init__(self, path: str):
        from safetensors import safe_open

        self.path = path
        self.safe_open = safe_open
        idx = os.path.join(path, "model.safetensors.index.json")
        if os.path.exists(idx):
            self.weight_map = json.load(open(idx))["weight_map"]
        else:
            self.weight_map = {}
            for fn in sorted(os.listdir(path)):
                if fn.endswith(".safetensors"):
                    with safe_open(os.path.join(path, fn), framework="pt") as f:
                        for k in f.keys():
                            self.weight_map[k] = fn
        self._open: dict[str, object] = {}

    def get(self, name: str) -> Optional[torch.Tensor]:
        fn = self.weight_map.get(name)
        if fn is None:
            return None
        h = self._open.get(fn)
        if h is None:
            h = self.safe_open(os.path.join(self.path, fn), framework="pt")
            self._open[fn] = h
        return h.get_tensor(name)


def load_pretrained(path: str, device="cpu", dtype: Optional[torch.dtype] = None, strict: bool = True, tp=None, ep=None,
                    pp_rank: int = 0, pp_size: int = 1, lora: Optional[dict] = None, vpp: int = 1, **cfg_overrides) -> CausalLM:
    """Builds a model (or this rank's tensor / expert / pipeline shard of it) from an HF checkpoint directory."""
    cfg = ModelConfig.from_pretrained(path, **cfg_overrides)
    from .transformer import build_model

    model = build_model(cfg, dtype=dtype, device=device, init=False, tp=tp, ep=ep, pp_rank=pp_rank, pp_size=pp_size, lora=lora, vpp=vpp)
    if lora:
        from .transformer import LoRA

        for name, mod in model.named_modules():
            if isinstance(mod, LoRA):
                g = torch.Generator(device=mod.lora_A.device)
                g.manual_seed(hash(name) & 0x7FFFFFFF)
                mod.reset(g)
        if os.path.exists(os.path.join(path, "adapter_model.safetensors")):
            load_lora_adapter(model, path)
    reader = _SafetensorsDir(path)
    get = reader.get
    if cfg.tie_word_embeddings or cfg.value_head:
        pass
    missing = load_hf_tensors(model, get, strict=False)
    # a value model initialised from a causal LM has no score.weight yet: start it at zero
    really_missing = [m for m in missing if not m.startswith("score.")]
    if strict and really_missing:
        raise KeyError(f"tensors missing from {path}: {really_missing[:5]}")
    if cfg.value_head and "score.weight" in missing:
        with torch.no_grad():
            model.score.zero_()
    return model


# --------------------------------------------------------------------------------------------- LoRA adapters (PEFT layout)
def iter_lora_tensors(model: CausalLM) -> Iterator[tuple[str, torch.Tensor]]:
    """(PEFT tensor name, view) for every enabled adapter: ``base_model.model.<hf module>.lora_{A,B}.weight``."""
    from .transformer import LoRA

    for mod_name, mod in model.named_modules():
        if not isinstance(mod, LoRA):
            continue
        li = model.layer_ids[int(mod_name.split(".")[1])]
        parent = "self_attn" if ".self_attn." in mod_name else "mlp"
        row = 0
        for s, (seg, n) in enumerate(mod.segments):
            if mod.enabled[s]:
                base = f"base_model.model.model.layers.{li}.{parent}.{seg}"
                yield f"{base}.lora_A.weight", mod.lora_A[s * mod.r : (s + 1) * mod.r]
                yield f"{base}.lora_B.weight", mod.lora_B[row : row + n]
            row += n


def save_lora_adapter(model: CausalLM, path: str) -> None:
    """Writes ``adapter_model.safetensors`` + ``adapter_config.json`` (the files PEFT loads)."""
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    sd = {n: t.detach().cpu().contiguous() for n, t in iter_lora_tensors(model)}
    save_file(sd, os.path.join(path, "adapter_model.safetensors"), metadata={"format": "pt"})
    c = model.lora_cfg or {}
    targets = sorted({n.split(".")[-3] for n in sd})
    with open(os.path.join(path, "adapter_config.json"), "w") as f:
        json.dump({"peft_type": "LORA", "r": int(c.get("dim", 8)), "lora_alpha": float(c.get("alpha", 32)), "lora_dropout": 0.0,
                   "target_modules": targets, "bias": "none", "task_type": "CAUSAL_LM"}, f, indent=2)


@torch.no_grad()
def load_lora_adapter(model: CausalLM, path: str) -> None:
    from safetensors import safe_open

    fn = os.path.join(path, "adapter_model.safetensors")
    with safe_open(fn, framework="pt") as f:
        have = set(f.keys())
        for n, dst in iter_lora_tensors(model):
            if n in have:
                dst.copy_(f.get_tensor(n).to(dst.dtype))


@torch.no_grad()
def merge_lora(model: CausalLM) -> CausalLM:
    """Folds every adapter into its base weight (W += scale * B A) and switches the adapters off: the model then
    behaves identically without them (export to a plain HF checkpoint, merged serving)."""
    for layer in model.layers:
        for owner, wname, lname in ((layer.self_attn, "qkv_proj", "qkv_lora"), (layer.self_attn, "o_proj", "o_lora"),
                                    (layer.mlp, "gate_up_proj", "gate_up_lora"), (layer.mlp, "down_proj", "down_lora")):
            lora = getattr(owner, lname, None)
            if lora is not None:
                w = getattr(owner, wname)
                w.copy_(model.merged_weight(w, lora))
                lora.lora_B.zero_()
    return model
