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


def _nemotron_get(sd):
    """HF keeps the experts stacked (``experts.up_proj`` [E, f, d]); checkpoints and this repo name them per expert."""
    import re

    def get(name):
        m = re.match(r"(.*\.mixer\.experts)\.(\d+)\.(up|down)_proj\.weight", name)
        return sd[f"{m.group(1)}.{m.group(3)}_proj"][int(m.group(2))] if m else sd.get(name)

    return get


@pytest.mark.parametrize("latent", [None, 24])
def test_nemotron_h_matches_huggingface(latent):
    """Nemotron-H: Mamba-2 mixers (chunked scan, depth-wise conv, grouped gated norm), attention without rotation, experts
    without a gate (squared ReLU) behind a sigmoid group-limited router, optionally in a latent space, plus a shared expert."""
    transformers = pytest.importorskip("transformers")
    if not hasattr(transformers, "NemotronHForCausalLM"):
        pytest.skip("this transformers build has no NemotronH")
    from rl_b200.models.config import ModelConfig
    from rl_b200.models.hf_io import iter_hf_tensors, load_hf_tensors
    from rl_b200.models.transformer import PackedBatch, build_model

    hf_cfg = transformers.NemotronHConfig(
        vocab_size=256, hidden_size=64, layers_block_type=["mamba", "moe", "attention", "mamba", "moe"], num_attention_heads=4,
        num_key_value_heads=2, head_dim=16, mamba_num_heads=8, mamba_head_dim=16, ssm_state_size=16, n_groups=2, chunk_size=8,
        n_routed_experts=4, moe_intermediate_size=32, moe_shared_expert_intermediate_size=48, num_experts_per_tok=2,
        moe_latent_size=latent, attn_implementation="eager", n_group=2, topk_group=1, routed_scaling_factor=1.5)
    torch.manual_seed(0)
    hf = transformers.NemotronHForCausalLM(hf_cfg).eval().float()
    for mod in hf.modules():      # the library's pure-PyTorch path clamps the step size at time_step_min; its kernels do not
        if hasattr(mod, "time_step_min"):
            mod.time_step_min = 0.0
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "norm" in n or n.endswith(".D"):
                p.copy_(1 + torch.randn_like(p) * 0.2)
            if "experts" in n or "gate.weight" in n:
                p.copy_(torch.randn_like(p) * 0.1)
        for n, b in hf.named_buffers():
            if "e_score" in n:
                b.copy_(torch.randn_like(b) * 0.1)
    cfg = ModelConfig.from_hf_dict(hf_cfg.to_dict(), torch_dtype="float32")
    assert cfg.is_hybrid and cfg.layers_block_type[0] == "mamba" and not cfg.use_rope and not cfg.mlp_gated and cfg.num_experts == 4
    assert ModelConfig.from_hf_dict(cfg.to_hf_dict()) == cfg
    m = build_model(cfg, dtype=torch.float32, init=False)
    sd = _hf_state(hf)
    assert not load_hf_tensors(m, _nemotron_get(sd))
    ids = torch.randint(0, 256, (2, 37))
    lens = torch.tensor([37, 21])       # several chunks of 8, one ragged
    with torch.no_grad():
        ref = hf(input_ids=ids, attention_mask=(torch.arange(37)[None] < lens[:, None]).long()).logits
        batch = PackedBatch.from_padded(ids, lens)
        z = batch.unpack(m.logits(batch), 37)
    for b, n in enumerate(lens.tolist()):
        assert (z[b, :n] - ref[b, :n]).abs().max().item() < 2e-4, (b, (z[b, :n] - ref[b, :n]).abs().max().item())
    out = dict(iter_hf_tensors(m))
    get = _nemotron_get(sd)
    for k, v in out.items():
        assert torch.allclose(v, get(k), atol=1e-6), k
    lp, _ = m.next_token_logprobs(batch)
    lp.sum().backward()
    skip = ("e_score",)
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for n, p in m.named_parameters() if not any(s in n for s in skip))


def test_mamba_mixer_continues_from_its_state():
    """A sequence evaluated in two pieces, and then token by token, gives what one pass gives: the states handed on (last conv
    inputs, state-space state) carry everything the rest of the sequence needs."""
    from rl_b200.models.config import ModelConfig
    from rl_b200.models.mamba import Mamba2Mixer

    cfg = ModelConfig(model_type="nemotron_h", hidden_size=32, layers_block_type=["mamba"], num_hidden_layers=1, mamba_num_heads=4,
                      mamba_head_dim=8, ssm_state_size=8, mamba_n_groups=2, mamba_chunk_size=4, use_rope=False, mlp_gated=False)
    torch.manual_seed(1)
    mx = Mamba2Mixer(cfg, torch.float32, "cpu")
    with torch.no_grad():
        for p in mx.parameters():
            p.copy_(torch.randn_like(p) * 0.3)
        mx.reset_special(torch.Generator().manual_seed(0))
    lens = [11, 6]
    u = torch.randn(sum(lens), 32)
    cu = torch.tensor([0, 11, 17], dtype=torch.int32)
    with torch.no_grad():
        full, (conv, ssm) = mx(u, cu, 11, return_state=True)
        # first 7 / 4 tokens, then the rest from the returned state
        a = torch.cat([u[0:7], u[11:15]])
        b = torch.cat([u[7:11], u[15:17]])
        ya, st = mx(a, torch.tensor([0, 7, 11], dtype=torch.int32), 7, return_state=True)
        yb, (conv2, ssm2) = mx(b, torch.tensor([0, 4, 6], dtype=torch.int32), 4, state=st, return_state=True)
        assert torch.allclose(torch.cat([ya[:7], yb[:4], ya[7:], yb[4:]]), full, atol=1e-5)
        assert torch.allclose(conv2, conv, atol=1e-6) and torch.allclose(ssm2, ssm, atol=1e-5)
        # token by token from the state after the first piece
        cs, ss = st
        outs = []
        for t in range(4):
            row = torch.stack([u[7 + t], u[15 + min(t, 1)]])
            y, cs, ss = mx.step(row, cs, ss)
            outs.append(y)
        assert torch.allclose(torch.stack([o[0] for o in outs]), full[7:11], atol=1e-5)
        assert torch.allclose(outs[0][1], full[15], atol=1e-5) and torch.allclose(outs[1][1], full[16], atol=1e-5)
