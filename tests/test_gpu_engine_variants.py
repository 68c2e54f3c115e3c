"""GPU checks of the newer engine paths: head dimensions other than 128 (gather fallback of the decode attention), low-precision
rollout (MXFP8 block-scaled GEMM, FP8 block-128 weights) and vision-language training + generation."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _gen_and_score(mc, gen_over=None, B=8, P=24, new=12):
    from rl_b200.distributed.batched_data_dict import BatchedDataDict
    from rl_b200.policy.worker import PolicyWorker

    g = dict(max_new_tokens=new, stop_token_ids=[], kv_cache_tokens=8192, block_size=16, max_running=32)
    g.update(gen_over or {})
    p = PolicyWorker(dict(precision="bfloat16", train_global_batch_size=8, train_micro_batch_size=4, max_total_sequence_length=256,
                          optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=1e-4)), generation=g),
                     model_cfg=mc, device="cuda:0", init_reference_model=False, seed=3)
    gen = p.build_generation()
    gen.prepare_for_generation()
    torch.manual_seed(0)
    ids = torch.randint(1, mc.vocab_size - 1, (B, P))
    out = gen.generate(BatchedDataDict(input_ids=ids, input_lengths=torch.full((B,), P)))
    data = BatchedDataDict(input_ids=out["output_ids"], input_lengths=out["unpadded_sequence_lengths"])
    lp = p.get_logprobs(data)["logprobs"]
    mask = out["logprobs"] != 0
    return (lp - out["logprobs"]).abs()[mask], out, gen


@pytest.mark.parametrize("graphs", [True, False])
def test_engine_with_head_dim_64_matches_trainer(graphs):
    from rl_b200.models.config import ModelConfig
    from rl_b200.ops.lib import check_status

    mc = ModelConfig(model_type="llama", vocab_size=4096, hidden_size=512, intermediate_size=1408, num_hidden_layers=2,
                     num_attention_heads=8, num_key_value_heads=4, head_dim=64, rope_theta=500000.0)
    err, out, _ = _gen_and_score(mc, dict(use_cuda_graphs=graphs))
    assert check_status() == 0 and (out["generation_lengths"] == 12).all()
    assert err.mean().item() < 0.03 and err.max().item() < 0.5


@pytest.mark.parametrize("kind", ["mxfp8", "fp8"])
def test_quantized_rollout_runs_and_stays_close(kind):
    from rl_b200.models.config import ModelConfig
    from rl_b200.ops.lib import check_status

    mc = ModelConfig(model_type="llama", vocab_size=4096, hidden_size=512, intermediate_size=1536, num_hidden_layers=2,
                     num_attention_heads=4, num_key_value_heads=2, head_dim=128, rope_theta=500000.0)
    err, out, gen = _gen_and_score(mc, dict(precision=kind))
    assert check_status() == 0 and gen.last_quantization["tensors"] == 8
    assert gen.last_quantization["quantized_bytes"] < 0.6 * gen.last_quantization["bf16_bytes"]
    assert 0 < err.mean().item() < 0.3 and err.max().item() < 2.0     # a quantised policy: close to, not equal to, the bf16 one


def test_vlm_sft_and_generation_on_gpu(tmp_path):
    from rl_b200.algorithms import sft
    from rl_b200.data.datasets.vlm import ProcessedVLMDataset, SyntheticColourDataset
    from rl_b200.data.tokenizers import ByteTokenizer
    from rl_b200.models.config import preset

    tok = ByteTokenizer(512)
    mc = preset("tiny-vlm", vocab_size=512)
    train = ProcessedVLMDataset(SyntheticColourDataset(128, image_size=16, colours=["red", "blue"], seed=0), tok, 4, 511, True)
    cfg = {"sft": dict(max_num_steps=24, max_num_epochs=4, val_period=0, seed=0),
           "policy": dict(precision="bfloat16", train_global_batch_size=16, train_micro_batch_size=8, logprob_batch_size=8, max_total_sequence_length=128,
                          max_grad_norm=1.0, optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=2e-3, weight_decay=0.0)),
                          generation=dict(max_new_tokens=8, stop_token_ids=[], kv_cache_tokens=8192, block_size=16, max_running=32)),
           "logger": dict(log_dir=str(tmp_path)), "checkpointing": dict(enabled=False), "data": dict(shuffle=True)}
    policy, loader, _, loss_fn, logger, ck, ss, cfg = sft.setup_sft(cfg, tok, train, None, model_cfg=mc)
    hist = []
    sft.sft_train(policy, loader, None, tok, loss_fn, logger, ck, ss, cfg, step_callback=lambda s, m: hist.append(m["train"]["loss"]))
    assert hist[-1] < 0.5 * hist[0]
    # generation with images: the engine's log-probabilities agree with the trainer's on the same images
    from rl_b200.data.collate import rl_collate_fn
    from rl_b200.data.llm_message_utils import batched_message_log_to_flat_message, multimodal_fields
    from rl_b200.distributed.batched_data_dict import BatchedDataDict

    prompts = ProcessedVLMDataset(SyntheticColourDataset(8, image_size=16, seed=5), tok, 4, 511, False)
    batch = rl_collate_fn([prompts[i] for i in range(8)])
    flat, lens = batched_message_log_to_flat_message(batch["message_log"], {"token_ids": tok.pad_token_id})
    gen = policy.build_generation()
    gen.prepare_for_generation()
    out = gen.generate(BatchedDataDict(input_ids=flat["token_ids"], input_lengths=lens, **multimodal_fields(flat)))
    assert not (out["output_ids"][:, int(lens.max()):] == 511).any()
    data = BatchedDataDict(input_ids=out["output_ids"], input_lengths=out["unpadded_sequence_lengths"], **multimodal_fields(flat))
    lp = policy.get_logprobs(data)["logprobs"]
    mask = out["logprobs"] != 0
    assert (lp - out["logprobs"]).abs()[mask].mean().item() < 0.05


@pytest.mark.parametrize("D,Hq,Hkv,bs", [(128, 8, 2, 16), (64, 4, 4, 32)])
def test_fused_rope_kv_write_matches_fp32_reference(D, Hq, Hkv, bs):
    """The fused kernel against a plain PyTorch fp32 restatement: rotate q and k (rotate_half convention), scatter k and v."""
    from rl_b200.models.config import ModelConfig, rope_inv_freq
    from rl_b200.ops import engine_ops as E

    torch.manual_seed(0)
    T, nblk = 37, 12
    dev = torch.device("cuda", 0)
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device=dev, dtype=torch.bfloat16)
    pos = torch.randint(0, 500, (T,), device=dev, dtype=torch.int32)
    mc = ModelConfig(vocab_size=64, hidden_size=Hq * D, intermediate_size=64, num_hidden_layers=1, num_attention_heads=Hq, num_key_value_heads=Hkv, head_dim=D)
    inv = rope_inv_freq(mc, dev)
    slots = torch.randperm(nblk * bs, device=dev)[:T].to(torch.int64)
    slots[5] = -1                                       # a padding row: rotated, not written
    kc = torch.zeros(nblk, Hkv, bs, D, device=dev, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    x = qkv.float().view(T, Hq + 2 * Hkv, D)
    ang = pos.float()[:, None] * inv.float()[None, :]
    cos, sin = torch.cat([ang.cos(), ang.cos()], -1)[:, None], torch.cat([ang.sin(), ang.sin()], -1)[:, None]
    rot = torch.cat([-x[..., D // 2 :], x[..., : D // 2]], -1)
    want = x.clone()
    want[:, : Hq + Hkv] = (x * cos + rot * sin)[:, : Hq + Hkv]
    out = E.rope_kv_cache_write(qkv.clone(), pos, inv, slots, kc, vc, Hq, Hkv, D)
    torch.cuda.synchronize()
    assert (out.float().view(T, -1, D) - want).abs().max().item() < 0.04       # bf16 rounding of values up to ~4
    ok = slots >= 0
    blk, off = (slots[ok] // bs).long(), (slots[ok] % bs).long()
    assert torch.equal(kc[blk, :, off], out.view(T, -1, D)[ok][:, Hq : Hq + Hkv])
    assert torch.equal(vc[blk, :, off], qkv.view(T, -1, D)[ok][:, Hq + Hkv :])
    assert int((kc.abs().sum((1, 3)) > 0).sum()) == int(ok.sum())             # nothing else was touched


def test_engine_serves_hybrid_state_space_model_on_gpu():
    """Nemotron-H blocks on the GPU: Mamba-2 states per running sequence through prefill and windowed decode, attention
    blocks on the paged cache, MLP and expert blocks; the engine's log-probabilities agree with the trainer's."""
    from rl_b200.models.config import preset
    from rl_b200.ops.lib import check_status

    mc = preset("tiny-nemotron-h", vocab_size=4096, hidden_size=512, intermediate_size=1024, head_dim=128, num_attention_heads=4,
                num_key_value_heads=2)
    err, out, gen = _gen_and_score(mc, dict(use_cuda_graphs=True))
    assert check_status() == 0 and (out["generation_lengths"] == 12).all()
    assert err.mean().item() < 0.03 and err.max().item() < 0.5
