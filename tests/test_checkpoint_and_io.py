"""Checkpoint manager (atomic dirs, retention, resume) and HF safetensors round trip incl. MoE and fused projections."""

import json
import os

import pytest
import torch

from rl_b200.models.config import ModelConfig
from rl_b200.models.hf_io import iter_hf_tensors, load_pretrained, save_pretrained
from rl_b200.models.transformer import CausalLM, PackedBatch
from rl_b200.utils.checkpoint import CheckpointManager


def test_checkpoint_manager_retention_and_resume(tmp_path):
    cm = CheckpointManager(dict(enabled=True, checkpoint_dir=str(tmp_path), metric_name="val:accuracy", higher_is_better=True, keep_top_k=2))
    for step, acc in [(1, 0.1), (2, 0.9), (3, 0.5), (4, 0.2)]:
        tmp = cm.init_tmp_checkpoint(step, {"step": step, "val": {"accuracy": acc}}, {"a": 1})
        (tmp / "policy" / "weights").mkdir(parents=True)
        assert not (tmp_path / f"step_{step}").exists()
        cm.finalize_checkpoint(tmp)
    kept = sorted(p.name for p in tmp_path.iterdir())
    assert kept == ["step_2", "step_3", "step_4"]  # best two + the latest
    assert cm.get_latest_checkpoint_path().endswith("step_4")
    assert cm.get_best_checkpoint_path().endswith("step_2")
    assert cm.load_training_info()["step"] == 4
    paths = cm.get_resume_paths()
    assert paths["weights"] and paths["optimizer"] is None
    cm.begin_finalization(cm.init_tmp_checkpoint(5, {"step": 5, "val": {"accuracy": 1.0}}))
    cm.wait()
    assert (tmp_path / "step_5").exists() and not (tmp_path / "tmp_step_5").exists()


@pytest.mark.parametrize("kind", ["llama", "qwen2", "qwen3", "qwen3_moe", "value"])
def test_hf_roundtrip(tmp_path, kind):
    kw = dict(vocab_size=64, hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              head_dim=8, torch_dtype="float32")
    if kind == "qwen2":
        kw.update(model_type="qwen2", attention_bias=True, tie_word_embeddings=True)
    elif kind == "qwen3":
        kw.update(model_type="qwen3", qk_norm=True)
    elif kind == "qwen3_moe":
        kw.update(model_type="qwen3_moe", qk_norm=True, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=16)
    elif kind == "value":
        kw.update(value_head=True)
    mc = ModelConfig(**kw)
    m = CausalLM(mc, dtype=torch.float32, seed=2)
    names = [n for n, _ in iter_hf_tensors(m)]
    assert "model.layers.0.self_attn.k_proj.weight" in names and len(names) == len(set(names))
    save_pretrained(m, str(tmp_path), max_shard_bytes=20000)
    assert os.path.exists(tmp_path / "config.json")
    m2 = load_pretrained(str(tmp_path), dtype=torch.float32, **({"value_head": True} if kind == "value" else {}))
    ids = torch.randint(0, 64, (2, 10))
    b = PackedBatch.from_padded(ids, torch.tensor([10, 7]))
    if kind == "value":
        assert torch.allclose(m.values(b), m2.values(b), atol=1e-6)
    else:
        assert torch.allclose(m.logits(b), m2.logits(b), atol=1e-6)


def test_model_packed_equals_separate_sequences():
    mc = ModelConfig(vocab_size=50, hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                     head_dim=8, torch_dtype="float32")
    m = CausalLM(mc, dtype=torch.float32, seed=4)
    ids = torch.randint(0, 50, (3, 12))
    lens = torch.tensor([12, 5, 9])
    packed, _ = m.next_token_logprobs(PackedBatch.from_padded(ids, lens))
    out = PackedBatch.from_padded(ids, lens).unpack(packed, 12)
    for i in range(3):
        one, _ = m.next_token_logprobs(PackedBatch.from_padded(ids[i : i + 1, : lens[i]], lens[i : i + 1]))
        assert torch.allclose(out[i, : lens[i]], one, atol=1e-5)
        assert out[i, 0] == 0


@pytest.mark.parametrize("stacked,arch", [(False, "llama"), (True, "qwen3"), (False, "moe")])
def test_megatron_checkpoint_converts_to_hf(tmp_path, stacked, arch):
    """A Megatron-core style distributed checkpoint (grouped qkv, fused gate / up, norms folded into the linear layers' names,
    experts by index; per-layer keys or one key per kind with a leading layer axis) becomes the HF checkpoint it came from."""
    import sys

    import torch.distributed.checkpoint as dcp

    from rl_b200.checkpoint import megatron_names as M
    from rl_b200.models.config import ModelConfig
    from rl_b200.models.hf_io import iter_hf_tensors, load_pretrained
    from rl_b200.models.transformer import build_model

    base = dict(vocab_size=96, hidden_size=32, intermediate_size=48, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2, head_dim=8,
                torch_dtype="float32")
    cfg = {"llama": ModelConfig(model_type="llama", **base),
           "qwen3": ModelConfig(model_type="qwen3", qk_norm=True, **base),
           "moe": ModelConfig(model_type="qwen3_moe", qk_norm=True, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=16, **base)}[arch]
    model = build_model(cfg, dtype=torch.float32, seed=4)
    hf = {k: v.detach().clone() for k, v in iter_hf_tensors(model)}
    q, k, v = (hf[f"model.layers.1.self_attn.{n}_proj.weight"] for n in "qkv")
    merged = M.merge_qkv(q, k, v, cfg)
    assert torch.equal(merged[:16], q[:16]) and torch.equal(merged[16:24], k[:8]) and torch.equal(merged[24:32], v[:8])      # group 0: 2 q heads, k, v
    assert all(torch.equal(a, b) for a, b in zip(M.split_qkv(merged, cfg), (q, k, v)))
    meg = M.hf_to_megatron(hf, cfg)
    if stacked:      # homogeneous stack: one entry per kind with a leading layer axis, under a "model." prefix
        kinds = {}
        for key, t in meg.items():
            m = __import__("re").match(r"decoder\.layers\.(\d+)\.(.*)", key)
            if m:
                kinds.setdefault(m.group(2), {})[int(m.group(1))] = t
        meg = {k_: t for k_, t in meg.items() if not k_.startswith("decoder.layers.")}
        meg.update({f"decoder.layers.{rest}": torch.stack([ts[i] for i in range(3)]) for rest, ts in kinds.items()})
        meg = {"model." + k_: t for k_, t in meg.items()}
    ck = tmp_path / "meg" / "iter_0000005"
    dcp.save({k_: t.contiguous() for k_, t in meg.items()}, checkpoint_id=str(ck), no_dist=True)
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from examples.converters import convert_megatron_to_hf as conv

    cfg.save_pretrained(str(tmp_path / "cfg"))
    conv.main(["--megatron-ckpt-path", str(tmp_path / "meg"), "--hf-config", str(tmp_path / "cfg"), "--hf-ckpt-path", str(tmp_path / "hf")])
    back = load_pretrained(str(tmp_path / "hf"), dtype=torch.float32)
    for (n, a), (_, b) in zip(model.named_parameters(), back.named_parameters()):
        assert torch.equal(a, b), n
