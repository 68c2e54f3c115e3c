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
