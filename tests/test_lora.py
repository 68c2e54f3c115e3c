"""LoRA: adapters train while the base stays frozen, the reference policy is the base model, adapters round-trip through
the PEFT file layout, and merging reproduces the adapted model."""

import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def _data():
    from rl_b200.distributed.batched_data_dict import BatchedDataDict

    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 2048, (8, 16), generator=g)
    return BatchedDataDict(input_ids=ids, input_lengths=torch.full((8,), 16), token_mask=torch.ones(8, 16), sample_mask=torch.ones(8))


def test_lora_training_merge_and_export(tmp_path):
    from rl_b200.algorithms.loss.loss_functions import NLLLossFn
    from rl_b200.models.config import preset
    from rl_b200.models.hf_io import load_pretrained, merge_lora, save_lora_adapter, save_pretrained
    from rl_b200.models.transformer import PackedBatch
    from rl_b200.parallel.state import reset_parallel
    from rl_b200.policy.worker import PolicyWorker

    reset_parallel()
    mc = preset("tiny-llama-oracle", torch_dtype="float32")
    cfg = dict(precision="float32", train_global_batch_size=8, train_micro_batch_size=4, max_total_sequence_length=32, max_grad_norm=1.0,
               logprob_batch_size=4, optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=2e-2, weight_decay=0.0)),
               lora_cfg=dict(enabled=True, dim=8, alpha=16, target_modules=["q_proj", "v_proj", "down_proj"]))
    w = PolicyWorker(cfg, model_cfg=mc, init_reference_model=True, seed=3)
    assert w.flat_base is not None and w.ref_flat is None
    n_train = sum(p.numel() for p in w.flat.params)
    n_base = sum(p.numel() for p in w.flat_base.params)
    assert n_train < 0.1 * n_base and all(not p.requires_grad for p in w.flat_base.params)
    base_before = w.flat_base.flat.clone()
    data = _data()
    lp0 = w.get_logprobs(data)["logprobs"]
    assert torch.allclose(lp0, w.get_reference_policy_logprobs(data)["reference_logprobs"])  # B = 0 at the start
    losses = [float(w.train(data, NLLLossFn(), gbs=8, mbs=4)["loss"][0]) for _ in range(8)]
    assert losses[-1] < losses[0] - 0.05, losses
    assert torch.equal(w.flat_base.flat, base_before)                       # the base never moves
    lp1 = w.get_logprobs(data)["logprobs"]
    ref = w.get_reference_policy_logprobs(data)["reference_logprobs"]
    assert torch.allclose(ref, lp0, atol=1e-6) and (lp1 - lp0).abs().max() > 1e-3
    # disabled segments stay untouched
    lora = w.model.layers[0].self_attn.qkv_lora
    assert lora.lora_B[mc.q_size : mc.q_size + mc.kv_size].abs().max() == 0 and lora.lora_B[: mc.q_size].abs().max() > 0
    # PEFT round trip + merge
    save_pretrained(w.model, str(tmp_path / "base"))
    save_lora_adapter(w.model, str(tmp_path / "base"))
    assert os.path.exists(tmp_path / "base" / "adapter_config.json")
    again = load_pretrained(str(tmp_path / "base"), dtype=torch.float32, lora=cfg["lora_cfg"])
    batch = PackedBatch.from_padded(data["input_ids"], data["input_lengths"])
    with torch.no_grad():
        z = w.model.logits(batch)
        assert torch.allclose(again.logits(batch), z, atol=1e-5)
        merged = merge_lora(again)
        merged.set_adapters(False)
        assert torch.allclose(merged.logits(batch), z, atol=1e-4)
    from examples.converters import convert_lora_to_hf

    convert_lora_to_hf.main(["--base-ckpt", str(tmp_path / "base"), "--adapter", str(tmp_path / "base"), "--out", str(tmp_path / "merged")])
    plain = load_pretrained(str(tmp_path / "merged"), dtype=torch.float32)
    with torch.no_grad():
        assert torch.allclose(plain.logits(batch), z, atol=1e-4)
