"""Model families against the HuggingFace implementations (fp32, CPU): same weights, same tokens, same logits."""

import pytest
import torch


def _hf_state(model):
    return {k: v.detach().clone() for k, v in model.state_dict().items()}


def test_gemma3_matches_huggingface():
    """Gemma 3 (text): tanh-GELU gate, norms before and after every block with (1 + w) weights, scaled embeddings, q/k norms,
    sliding-window layers with their own RoPE base, a global layer with linearly scaled RoPE, tied output head."""
    transformers = pytest.importorskip("transformers")
    from rl_b200.models.config import ModelConfig
    from rl_b200.models.hf_io import iter_hf_tensors, load_hf_tensors
    from rl_b200.models.transformer import PackedBatch, build_model

    hf_cfg = transformers.Gemma3TextConfig(vocab_size=512, hidden_size=64, intermediate_size=160, num_hidden_layers=6, num_attention_heads=4,
                                           num_key_value_heads=2, head_dim=32, sliding_window=8, query_pre_attn_scalar=24,
                                           max_position_embeddings=256, rms_norm_eps=1e-6, attn_implementation="eager")
    torch.manual_seed(0)
    hf = transformers.Gemma3ForCausalLM(hf_cfg).eval().float()
    with torch.no_grad():   # norms initialise to zero offset: give them something to get wrong
        for n, p in hf.named_parameters():
            if "norm" in n:
                p.copy_(torch.randn_like(p) * 0.2)
    cfg = ModelConfig.from_hf_dict(hf_cfg.to_dict(), torch_dtype="float32")
    assert cfg.model_type == "gemma3_text" and cfg.sandwich_norm and cfg.qk_norm and cfg.tie_word_embeddings
    assert cfg.layer_types.count("full_attention") == 1 and cfg.layer_is_sliding(0) and not cfg.layer_is_sliding(5)
    assert cfg.attn_scale == pytest.approx(24 ** -0.5) and cfg.embed_scale == pytest.approx(8.0) and cfg.rope_local_theta == 10000.0
    m = build_model(cfg, dtype=torch.float32, init=False)
    sd = _hf_state(hf)
    missing = load_hf_tensors(m, sd.get)
    assert not missing
    ids = torch.randint(0, 512, (2, 40))
    lens = torch.tensor([40, 23])          # both longer than the window of 8
    with torch.no_grad():
        ref = hf(input_ids=ids, attention_mask=(torch.arange(40)[None] < lens[:, None]).long()).logits
        batch = PackedBatch.from_padded(ids, lens)
        z = batch.unpack(m.logits(batch), 40)
    for b, n in enumerate(lens.tolist()):
        assert (z[b, :n] - ref[b, :n]).abs().max().item() < 2e-4, (b, (z[b, :n] - ref[b, :n]).abs().max().item())
    # the way back: exported tensors equal the checkpoint's (norm weights in their stored w - 1 form)
    out = dict(iter_hf_tensors(m))
    for k, v in sd.items():
        if k == "lm_head.weight":
            continue    # tied
        assert torch.allclose(out[k], v, atol=1e-6), k
    # training works through the same layers
    lp, _ = m.next_token_logprobs(batch)
    lp.sum().backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for n, p in m.named_parameters())


def _deepseek_get(sd):
    """HF keeps the experts stacked (``experts.gate_up_proj`` [E, 2f, d]); checkpoints and this repo name them per expert."""
    import re

    def get(name):
        m = re.match(r"(.*\.mlp\.experts)\.(\d+)\.(gate|up|down)_proj\.weight", name)
        if not m:
            return sd.get(name)
        base, e, which = m.group(1), int(m.group(2)), m.group(3)
        if which == "down":
            return sd[base + ".down_proj"][e]
        gu = sd[base + ".gate_up_proj"][e]
        f = gu.shape[0] // 2
        return gu[:f] if which == "gate" else gu[f:]

    return get


@pytest.mark.parametrize("q_lora,yarn", [(24, False), (None, True)])
def test_deepseek_v3_matches_huggingface(q_lora, yarn):
    """DeepSeek-V3: latent attention with the decoupled, interleaved rotary part, a dense first layer, then experts chosen by
    sigmoid score + bias inside the best groups, weighted by the renormalised, scaled scores, plus a shared expert."""
    transformers = pytest.importorskip("transformers")
    from rl_b200.models.config import ModelConfig
    from rl_b200.models.hf_io import iter_hf_tensors, load_hf_tensors
    from rl_b200.models.transformer import PackedBatch, build_model

    rope = dict(rope_type="yarn", factor=4.0, original_max_position_embeddings=64, beta_fast=32, beta_slow=1, mscale=1.0, mscale_all_dim=1.0,
                rope_theta=10000.0) if yarn else None
    hf_cfg = transformers.DeepseekV3Config(vocab_size=512, hidden_size=64, intermediate_size=128, moe_intermediate_size=32, num_hidden_layers=3,
                                           num_attention_heads=4, num_key_value_heads=4, n_routed_experts=8, n_shared_experts=1, num_experts_per_tok=3, n_group=4,
                                           topk_group=2, first_k_dense_replace=1, kv_lora_rank=16, q_lora_rank=q_lora, qk_nope_head_dim=16,
                                           qk_rope_head_dim=8, v_head_dim=12, routed_scaling_factor=2.5, max_position_embeddings=256,
                                           rope_parameters=rope, attn_implementation="eager")
    torch.manual_seed(0)
    hf = transformers.DeepseekV3ForCausalLM(hf_cfg).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "norm" in n:
                p.add_(torch.randn_like(p) * 0.2)
            elif p.dim() >= 2:
                p.normal_(0, 0.08)
        for n, b in hf.named_buffers():
            if n.endswith("e_score_correction_bias"):
                b.copy_(torch.randn_like(b) * 0.3)
    cfg = ModelConfig.from_hf_dict(hf_cfg.to_dict(), torch_dtype="float32")
    assert cfg.is_mla and cfg.head_dim == 24 and cfg.num_experts == 8 and cfg.scoring_func == "sigmoid" and not cfg.layer_is_moe(0) and cfg.layer_is_moe(1)
    m = build_model(cfg, dtype=torch.float32, init=False)
    sd = _hf_state(hf)
    sd.update({n: b.detach().clone() for n, b in hf.named_buffers() if n.endswith("e_score_correction_bias")})
    assert not load_hf_tensors(m, _deepseek_get(sd))
    ids = torch.randint(0, 512, (2, 100 if yarn else 30))
    S = ids.shape[1]
    lens = torch.tensor([S, S - 11])
    with torch.no_grad():
        ref = hf(input_ids=ids, attention_mask=(torch.arange(S)[None] < lens[:, None]).long()).logits
        batch = PackedBatch.from_padded(ids, lens)
        z = batch.unpack(m.logits(batch), S)
    for b, n in enumerate(lens.tolist()):
        assert (z[b, :n] - ref[b, :n]).abs().max().item() < 3e-4, (b, (z[b, :n] - ref[b, :n]).abs().max().item())
    out = dict(iter_hf_tensors(m))
    get = _deepseek_get(sd)
    assert all(torch.equal(t, get(k)) for k, t in out.items())
    lp, _ = m.next_token_logprobs(batch)
    lp.sum().backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for n, p in m.named_parameters())


@pytest.mark.parametrize("family", ["gemma3", "deepseek_v3"])
def test_saved_checkpoints_load_in_huggingface(tmp_path, family):
    """The way out: a checkpoint written by ``save_pretrained`` is read by ``AutoModelForCausalLM.from_pretrained`` (config and
    tensor names included) and produces the same logits."""
    transformers = pytest.importorskip("transformers")
    from rl_b200.models.config import ModelConfig
    from rl_b200.models.hf_io import save_pretrained
    from rl_b200.models.transformer import PackedBatch, build_model

    if family == "gemma3":
        hc = transformers.Gemma3TextConfig(vocab_size=512, hidden_size=64, intermediate_size=160, num_hidden_layers=6, num_attention_heads=4,
                                           num_key_value_heads=2, head_dim=32, sliding_window=8, query_pre_attn_scalar=24, max_position_embeddings=256)
    else:
        hc = transformers.DeepseekV3Config(vocab_size=512, hidden_size=64, intermediate_size=128, moe_intermediate_size=32, num_hidden_layers=3,
                                           num_attention_heads=4, num_key_value_heads=4, n_routed_experts=8, n_shared_experts=1,
                                           num_experts_per_tok=2, n_group=2, topk_group=1, first_k_dense_replace=1, kv_lora_rank=16, q_lora_rank=24,
                                           qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16, max_position_embeddings=256)
    cfg = ModelConfig.from_hf_dict(hc.to_dict(), torch_dtype="float32")
    m = build_model(cfg, dtype=torch.float32, seed=3)
    save_pretrained(m, str(tmp_path))
    hf = transformers.AutoModelForCausalLM.from_pretrained(str(tmp_path), dtype=torch.float32, attn_implementation="eager").eval()
    ids = torch.randint(0, 512, (1, 24))
    with torch.no_grad():
        ref = hf(input_ids=ids).logits[0]
        z = m.logits(PackedBatch.from_padded(ids, torch.tensor([24])))
    assert (z - ref).abs().max().item() < 1e-5


def _family_config(transformers, family):
    common = dict(vocab_size=512, hidden_size=64, intermediate_size=160, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                  max_position_embeddings=512, attn_implementation="eager")
    if family == "llama":
        return transformers.LlamaConfig(**common, rope_parameters=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                                                      original_max_position_embeddings=64, rope_theta=500000.0))
    if family == "mistral":
        return transformers.MistralConfig(**common, sliding_window=None)
    if family == "qwen2":
        return transformers.Qwen2Config(**common, tie_word_embeddings=True)
    if family == "qwen3":
        return transformers.Qwen3Config(**common, head_dim=32)
    if family == "qwen3_moe":
        return transformers.Qwen3MoeConfig(**common, head_dim=32, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=48, norm_topk_prob=True,
                                           decoder_sparse_step=1, mlp_only_layers=[])
    raise KeyError(family)


@pytest.mark.parametrize("family", ["llama", "mistral", "qwen2", "qwen3", "qwen3_moe"])
def test_dense_and_moe_families_match_huggingface(tmp_path, family):
    """Same check for the families the benchmarks use: our checkpoint, HuggingFace's model class, equal logits on a sequence
    long enough to reach the scaled part of the RoPE spectrum."""
    transformers = pytest.importorskip("transformers")
    from rl_b200.models.config import ModelConfig
    from rl_b200.models.hf_io import save_pretrained
    from rl_b200.models.transformer import PackedBatch, build_model

    hc = _family_config(transformers, family)
    d = hc.to_dict()
    if "rope_parameters" in d and isinstance(d["rope_parameters"], dict):     # newer configs nest what older ones spell rope_theta / rope_scaling
        rp = dict(d["rope_parameters"])
        d.setdefault("rope_theta", rp.pop("rope_theta", 10000.0))
        d["rope_theta"] = rp.pop("rope_theta", d["rope_theta"]) if "rope_theta" in rp else d["rope_theta"]
        d["rope_scaling"] = rp if rp.get("rope_type", "default") != "default" else None
    cfg = ModelConfig.from_hf_dict(d, torch_dtype="float32")
    m = build_model(cfg, dtype=torch.float32, seed=5)
    with torch.no_grad():
        for n, p in m.named_parameters():
            if "norm" in n:
                p.add_(torch.randn_like(p) * 0.1)
            elif n.endswith("bias"):
                p.normal_(0, 0.1)
    save_pretrained(m, str(tmp_path))
    hf = transformers.AutoModelForCausalLM.from_pretrained(str(tmp_path), dtype=torch.float32, attn_implementation="eager").eval()
    ids = torch.randint(0, 512, (1, 200))
    with torch.no_grad():
        ref = hf(input_ids=ids).logits[0]
        z = m.logits(PackedBatch.from_padded(ids, torch.tensor([200])))
    assert (z - ref).abs().max().item() < 2e-4, (family, (z - ref).abs().max().item())
