"""Megatron-core parameter names <-> HuggingFace names for the dense and mixture-of-experts decoder families, and the offline
conversion of a Megatron-core distributed checkpoint (a ``torch.distributed.checkpoint`` directory) to HF safetensors. Role of
examples/converters/convert_megatron_to_hf.py in the reference, which goes through Megatron-Bridge; here the mapping is written
out, so no Megatron installation is needed:

    embedding.word_embeddings.weight                         model.embed_tokens.weight
    decoder.layers.N.self_attention.linear_qkv.weight        q / k / v, interleaved per key-value group: [q heads of the group | k | v]
    decoder.layers.N.self_attention.linear_qkv.layer_norm_weight      input_layernorm
    decoder.layers.N.self_attention.{q,k}_layernorm.weight   q_norm / k_norm
    decoder.layers.N.self_attention.linear_proj.weight       o_proj
    decoder.layers.N.mlp.linear_fc1.weight                   [gate | up]           (layer_norm_weight: post_attention_layernorm)
    decoder.layers.N.mlp.linear_fc2.weight                   down_proj
    decoder.layers.N.pre_mlp_layernorm.weight                post_attention_layernorm (mixture layers)
    decoder.layers.N.mlp.router.weight                       mlp.gate.weight
    decoder.layers.N.mlp.experts.linear_fc{1,2}.weightE      experts.E.{gate,up,down}_proj
    decoder.final_layernorm.weight / output_layer.weight     model.norm / lm_head

Checkpoints of homogeneous stacks store the layers of one kind under ONE key with a leading layer axis
(``decoder.layers.self_attention.linear_qkv.weight`` of shape [L, ...]); both forms are read.
"""

from __future__ import annotations

import os
import re
from typing import Iterator

import torch

from rl_b200.models.config import ModelConfig


def split_qkv(qkv: torch.Tensor, cfg: ModelConfig) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Megatron's grouped layout -> separate q, k, v (works for weights [rows, d] and biases [rows])."""
    hd, nkv = cfg.head_dim, cfg.num_key_value_heads
    per = cfg.num_attention_heads // nkv
    g = qkv.reshape(nkv, (per + 2) * hd, *qkv.shape[1:])
    q = g[:, : per * hd].reshape(nkv * per * hd, *qkv.shape[1:])
    k = g[:, per * hd : (per + 1) * hd].reshape(nkv * hd, *qkv.shape[1:])
    v = g[:, (per + 1) * hd :].reshape(nkv * hd, *qkv.shape[1:])
    return q, k, v


def merge_qkv(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cfg: ModelConfig) -> torch.Tensor:
    hd, nkv = cfg.head_dim, cfg.num_key_value_heads
    per = cfg.num_attention_heads // nkv
    rest = q.shape[1:]
    return torch.cat([q.reshape(nkv, per * hd, *rest), k.reshape(nkv, hd, *rest), v.reshape(nkv, hd, *rest)], dim=1).reshape(-1, *rest)


def megatron_to_hf(state: dict[str, torch.Tensor], cfg: ModelConfig) -> Iterator[tuple[str, torch.Tensor]]:
    """Yields (HF name, tensor) for a Megatron-core state dictionary (per-layer keys; see :func:`unstack_layers`)."""
    def get(k):
        return state.get(k)

    if get("embedding.word_embeddings.weight") is not None:
        yield "model.embed_tokens.weight", state["embedding.word_embeddings.weight"][: cfg.vocab_size]
    if get("decoder.final_layernorm.weight") is not None:
        yield "model.norm.weight", state["decoder.final_layernorm.weight"]
    if get("output_layer.weight") is not None and not cfg.tie_word_embeddings:
        yield "lm_head.weight", state["output_layer.weight"][: cfg.vocab_size]
    for n in range(cfg.num_hidden_layers):
        mp, hp = f"decoder.layers.{n}", f"model.layers.{n}"
        qkv = get(f"{mp}.self_attention.linear_qkv.weight")
        if qkv is not None:
            for name, t in zip(("q_proj", "k_proj", "v_proj"), split_qkv(qkv, cfg)):
                yield f"{hp}.self_attn.{name}.weight", t
        b = get(f"{mp}.self_attention.linear_qkv.bias")
        if b is not None:
            for name, t in zip(("q_proj", "k_proj", "v_proj"), split_qkv(b, cfg)):
                yield f"{hp}.self_attn.{name}.bias", t
        for src, dst in ((f"{mp}.self_attention.linear_qkv.layer_norm_weight", f"{hp}.input_layernorm.weight"),
                         (f"{mp}.input_layernorm.weight", f"{hp}.input_layernorm.weight"),
                         (f"{mp}.self_attention.linear_proj.weight", f"{hp}.self_attn.o_proj.weight"),
                         (f"{mp}.self_attention.q_layernorm.weight", f"{hp}.self_attn.q_norm.weight"),
                         (f"{mp}.self_attention.k_layernorm.weight", f"{hp}.self_attn.k_norm.weight"),
                         (f"{mp}.mlp.linear_fc1.layer_norm_weight", f"{hp}.post_attention_layernorm.weight"),
                         (f"{mp}.pre_mlp_layernorm.weight", f"{hp}.post_attention_layernorm.weight"),
                         (f"{mp}.mlp.linear_fc2.weight", f"{hp}.mlp.down_proj.weight"),
                         (f"{mp}.mlp.router.weight", f"{hp}.mlp.gate.weight")):
            if get(src) is not None:
                yield dst, state[src]
        fc1 = get(f"{mp}.mlp.linear_fc1.weight")
        if fc1 is not None:
            yield f"{hp}.mlp.gate_proj.weight", fc1[: fc1.shape[0] // 2]
            yield f"{hp}.mlp.up_proj.weight", fc1[fc1.shape[0] // 2 :]
        for e in range(cfg.num_experts):
            w1, w2 = get(f"{mp}.mlp.experts.linear_fc1.weight{e}"), get(f"{mp}.mlp.experts.linear_fc2.weight{e}")
            if w1 is None:
                w1, w2 = get(f"{mp}.mlp.experts.local_experts.{e}.linear_fc1.weight"), get(f"{mp}.mlp.experts.local_experts.{e}.linear_fc2.weight")
            if w1 is not None:
                yield f"{hp}.mlp.experts.{e}.gate_proj.weight", w1[: w1.shape[0] // 2]
                yield f"{hp}.mlp.experts.{e}.up_proj.weight", w1[w1.shape[0] // 2 :]
                yield f"{hp}.mlp.experts.{e}.down_proj.weight", w2


def hf_to_megatron(hf: dict[str, torch.Tensor], cfg: ModelConfig) -> dict[str, torch.Tensor]:
    """The inverse mapping (dense and mixture layers), e.g. to hand HF weights to a Megatron-core job."""
    out = {"embedding.word_embeddings.weight": hf["model.embed_tokens.weight"], "decoder.final_layernorm.weight": hf["model.norm.weight"]}
    if "lm_head.weight" in hf:
        out["output_layer.weight"] = hf["lm_head.weight"]
    for n in range(cfg.num_hidden_layers):
        mp, hp = f"decoder.layers.{n}", f"model.layers.{n}"
        out[f"{mp}.self_attention.linear_qkv.weight"] = merge_qkv(hf[f"{hp}.self_attn.q_proj.weight"], hf[f"{hp}.self_attn.k_proj.weight"],
                                                                   hf[f"{hp}.self_attn.v_proj.weight"], cfg)
        if f"{hp}.self_attn.q_proj.bias" in hf:
            out[f"{mp}.self_attention.linear_qkv.bias"] = merge_qkv(hf[f"{hp}.self_attn.q_proj.bias"], hf[f"{hp}.self_attn.k_proj.bias"],
                                                                     hf[f"{hp}.self_attn.v_proj.bias"], cfg)
        out[f"{mp}.self_attention.linear_qkv.layer_norm_weight"] = hf[f"{hp}.input_layernorm.weight"]
        out[f"{mp}.self_attention.linear_proj.weight"] = hf[f"{hp}.self_attn.o_proj.weight"]
        for a, b in (("q_norm", "q_layernorm"), ("k_norm", "k_layernorm")):
            if f"{hp}.self_attn.{a}.weight" in hf:
                out[f"{mp}.self_attention.{b}.weight"] = hf[f"{hp}.self_attn.{a}.weight"]
        if f"{hp}.mlp.gate.weight" in hf:
            out[f"{mp}.pre_mlp_layernorm.weight"] = hf[f"{hp}.post_attention_layernorm.weight"]
            out[f"{mp}.mlp.router.weight"] = hf[f"{hp}.mlp.gate.weight"]
            for e in range(cfg.num_experts):
                out[f"{mp}.mlp.experts.linear_fc1.weight{e}"] = torch.cat([hf[f"{hp}.mlp.experts.{e}.gate_proj.weight"], hf[f"{hp}.mlp.experts.{e}.up_proj.weight"]])
                out[f"{mp}.mlp.experts.linear_fc2.weight{e}"] = hf[f"{hp}.mlp.experts.{e}.down_proj.weight"]
        else:
            out[f"{mp}.mlp.linear_fc1.layer_norm_weight"] = hf[f"{hp}.post_attention_layernorm.weight"]
            out[f"{mp}.mlp.linear_fc1.weight"] = torch.cat([hf[f"{hp}.mlp.gate_proj.weight"], hf[f"{hp}.mlp.up_proj.weight"]])
            out[f"{mp}.mlp.linear_fc2.weight"] = hf[f"{hp}.mlp.down_proj.weight"]
    return out


def unstack_layers(state: dict[str, torch.Tensor], num_layers: int) -> dict[str, torch.Tensor]:
    """``decoder.layers.<rest>`` entries with a leading layer axis become ``decoder.layers.N.<rest>``; ``model.`` / ``module.``
    prefixes and optimizer / RNG entries are dropped."""
    out = {}
    for k, v in state.items():
        k = re.sub(r"^(model\.|module\.)+", "", k)
        if not isinstance(v, torch.Tensor) or k.startswith(("optimizer", "rng", "opt_param_scheduler")) or k.endswith("._extra_state"):
            continue
        m = re.match(r"decoder\.layers\.(?!\d+\.)(.*)", k)
        if m and v.dim() >= 1 and v.shape[0] == num_layers:
            for n in range(num_layers):
                out[f"decoder.layers.{n}.{m.group(1)}"] = v[n]
        else:
            out[k] = v
    return out


def load_megatron_checkpoint(path: str) -> dict[str, torch.Tensor]:
    """All tensors of a Megatron-core distributed checkpoint directory (``.metadata`` + ``__*.distcp``; an ``iter_XXXXXXX`` parent is
    resolved to its newest iteration), single process."""
    import torch.distributed.checkpoint as dcp
    from torch.distributed.checkpoint import FileSystemReader
    from torch.distributed.checkpoint.metadata import TensorStorageMetadata

    if not os.path.exists(os.path.join(path, ".metadata")):
        its = sorted(d for d in os.listdir(path) if d.startswith("iter_") and os.path.exists(os.path.join(path, d, ".metadata")))
        if not its:
            raise FileNotFoundError(f"{path} is not a distributed checkpoint directory (no .metadata)")
        path = os.path.join(path, its[-1])
    md = FileSystemReader(path).read_metadata().state_dict_metadata
    state = {k: torch.zeros(tuple(m.size), dtype=m.properties.dtype) for k, m in md.items() if isinstance(m, TensorStorageMetadata)}
    dcp.load(state, checkpoint_id=path, no_dist=True)
    return state


def convert_megatron_to_hf(megatron_path: str, hf_path: str, model_cfg: ModelConfig) -> str:
    from rl_b200.models.hf_io import load_hf_tensors, save_pretrained
    from rl_b200.models.transformer import CausalLM

    state = unstack_layers(load_megatron_checkpoint(megatron_path), model_cfg.num_hidden_layers)
    tensors = dict(megatron_to_hf(state, model_cfg))
    dtype = next(t.dtype for t in tensors.values() if t.is_floating_point())
    model = CausalLM(model_cfg, dtype=dtype, device="cpu", init=False)
    with torch.no_grad():
        load_hf_tensors(model, tensors.get, strict=True)
    save_pretrained(model, hf_path)
    return hf_path
