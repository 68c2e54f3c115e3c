"""EAGLE-3 style draft head: module, checkpoint names, and training beside the policy through the worker."""

import os

import pytest
import torch

from rl_b200.models.config import preset


def _data():
    from rl_b200.distributed.batched_data_dict import BatchedDataDict

    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 2048, (8, 20), generator=g)
    lens = torch.tensor([20, 13, 17, 20, 9, 20, 15, 11])
    return BatchedDataDict(input_ids=ids, input_lengths=lens, token_mask=(torch.arange(20)[None] < lens[:, None]).float(), sample_mask=torch.ones(8))


def _cfg(**over):
    c = dict(precision="float32", train_global_batch_size=8, train_micro_batch_size=4, max_total_sequence_length=64, max_grad_norm=1.0,
             optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=3e-3)))
    c.update(over)
    return c


def test_aux_layers_and_checkpoint_names(tmp_path):
    from rl_b200.models.draft import EagleDraft, eagle3_aux_layers

    assert eagle3_aux_layers(32) == (1, 15, 28) and eagle3_aux_layers(4) == (1,) and eagle3_aux_layers(1) == (0,)
    mc = preset("tiny-llama-oracle", torch_dtype="float32", num_hidden_layers=12)
    d = EagleDraft(mc, dtype=torch.float32)
    assert d.aux_layers == (1, 5, 8) and d.fc.shape == (256, 3 * 256) and d.layers[0].self_attn.qkv_proj.shape[1] == 512
    sd = d.hf_state_dict()
    for k in ("fc.weight", "midlayer.hidden_norm.weight", "midlayer.self_attn.q_proj.weight", "midlayer.mlp.down_proj.weight", "lm_head.weight",
              "norm.weight", "d2t", "t2d"):
        assert k in sd, k
    assert sd["midlayer.self_attn.q_proj.weight"].shape == (mc.q_size, 512)
    d.save_pretrained(str(tmp_path / "draft"))
    d2 = EagleDraft(mc, dtype=torch.float32)
    d2.reset_parameters(seed=9)
    assert not torch.equal(d2.fc, d.fc)
    assert d2.load_pretrained(str(tmp_path / "draft")) == []
    for (n, a), (_, b) in zip(d.named_parameters(), d2.named_parameters()):
        assert torch.equal(a, b), n
    # a reduced draft vocabulary: ids map to policy tokens through offsets, the head starts as the policy's rows
    sub = EagleDraft(mc, draft_vocab_size=64, dtype=torch.float32)
    ids = torch.arange(0, 2048, 32)
    sub.set_vocab_subset(ids)
    assert torch.equal(sub.target_ids(), ids) and int(sub.t2d.sum()) == 64
    head = torch.randn(2048, 256)
    sub.init_head_from_policy(head)
    assert torch.equal(sub.lm_head.data, head[ids])
    T = 11
    out = sub(torch.randn(T, 3 * 256), torch.randn(T, 256), torch.arange(T, dtype=torch.int32), torch.ones(32), torch.tensor([0, 6, 11], dtype=torch.int32), 6)
    assert out.shape == (T, 64) and out.dtype == torch.float32


def test_draft_trains_beside_the_policy_and_leaves_it_alone(tmp_path):
    """The draft's loss falls and its agreement with the policy rises; the policy's own update is what it is without a draft
    (hidden states and targets are detached); the draft is saved beside the weights and comes back."""
    from rl_b200.algorithms.loss.loss_functions import NLLLossFn
    from rl_b200.policy.worker import PolicyWorker

    mc = preset("tiny-llama-oracle", torch_dtype="float32")
    data = _data()
    plain = PolicyWorker(_cfg(), model_cfg=mc, device="cpu", init_reference_model=False, seed=5)
    w = PolicyWorker(_cfg(draft=dict(enabled=True, loss_weight=0.5, num_layers=1)), model_cfg=mc, device="cpu", init_reference_model=False, seed=5)
    assert w.draft is not None and w.model.capture_layers == (1,)
    assert torch.equal(w.draft.lm_head.data, w.model.output_weight.data)      # head initialised from the policy's
    r0, rp = w.train(data, NLLLossFn()), plain.train(data, NLLLossFn())
    m = r0["all_mb_metrics"]
    assert "draft_loss" in m and "draft_accuracy" in m and "draft_grad_norm" in m and "policy_loss" in m
    # total = policy + 0.5 * draft on every micro-batch
    for tot, pl, dl in zip(m["loss"], m["policy_loss"], m["draft_loss"]):
        assert tot == pytest.approx(pl + 0.5 * dl, rel=1e-5)
    assert float(rp["grad_norm"][0]) == pytest.approx(float(r0["grad_norm"][0]), rel=1e-5)
    for (n, a), (_, b) in zip(w.model.named_parameters(), plain.model.named_parameters()):
        assert torch.allclose(a, b, atol=1e-7), n
    first = sum(m["draft_loss"])
    for _ in range(7):
        r = w.train(data, NLLLossFn())
    last = r["all_mb_metrics"]
    assert sum(last["draft_loss"]) < 0.85 * first and max(last["draft_accuracy"]) > 0.1
    path = str(tmp_path / "step_1" / "policy" / "weights")
    w.save_checkpoint(path)
    assert os.path.exists(str(tmp_path / "step_1" / "policy" / "draft" / "model.safetensors"))
    w2 = PolicyWorker(_cfg(draft=dict(enabled=True)), model_cfg=mc, device="cpu", init_reference_model=False, seed=77)
    w2.load_checkpoint(path)
    for (n, a), (_, b) in zip(w.draft.named_parameters(), w2.draft.named_parameters()):
        assert torch.equal(a, b), n
    # evaluation reports the draft's loss without touching it
    before = w.draft.fc.detach().clone()
    ev = w.train(data, NLLLossFn(), eval_mode=True)
    assert "draft_loss" in ev["all_mb_metrics"] and torch.equal(before, w.draft.fc)


def test_draft_refuses_layouts_it_does_not_cover():
    from rl_b200.models.draft import EagleDraft

    with pytest.raises(NotImplementedError):
        EagleDraft(preset("tiny-nemotron-h"))
