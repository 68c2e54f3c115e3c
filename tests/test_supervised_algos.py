"""SFT / DPO / RM loops on CPU with tiny models: losses fall and preference accuracy rises."""

import torch

from rl_b200.algorithms.sft import dpo_train, rm_train, setup_dpo, setup_rm, setup_sft, sft_train
from rl_b200.data.datasets.preference import RandomPreferenceDataset, RandomSFTDataset
from rl_b200.models.config import ModelConfig


def _mc(**kw):
    return ModelConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=8, torch_dtype="float32", **kw)


def _cfg(tmp_path, key, steps, **alg):
    return {
        key: dict(max_num_steps=steps, max_num_epochs=10, val_period=0, seed=0, **alg),
        "policy": dict(precision="float32", train_global_batch_size=16, train_micro_batch_size=8, logprob_batch_size=16,
                       max_total_sequence_length=64, max_grad_norm=1.0,
                       optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=5e-3, weight_decay=0.0)),
                       scheduler=[dict(name="torch.optim.lr_scheduler.LinearLR", kwargs=dict(start_factor=0.5, total_iters=5)),
                                  dict(name="torch.optim.lr_scheduler.ConstantLR", kwargs=dict(factor=1.0, total_iters=1000)),
                                  dict(milestones=[5])]),
        "logger": dict(log_dir=str(tmp_path / "logs")),
        "checkpointing": dict(enabled=True, checkpoint_dir=str(tmp_path / "ckpt"), save_period=1000, keep_top_k=2),
        "data": dict(shuffle=True),
    }


def test_sft_learns_and_checkpoints(tmp_path):
    ds = RandomSFTDataset(256, 64, seed=0)
    cfg = _cfg(tmp_path, "sft", 25)
    policy, loader, vl, loss_fn, logger, ck, ss, cfg = setup_sft(cfg, None, ds, RandomSFTDataset(32, 64, seed=1), model_cfg=_mc())
    hist = []
    sft_train(policy, loader, vl, None, loss_fn, logger, ck, ss, cfg, step_callback=lambda s, m: hist.append(m["train"]["loss"]))
    assert hist[-1] < 0.7 * hist[0], hist
    assert abs(policy.optimizer.lr - 5e-3) < 1e-9  # warm-up finished
    assert ck.get_latest_checkpoint_path().endswith("step_25")
    # resume restores weights, optimizer shard and dataloader position
    cfg2 = _cfg(tmp_path, "sft", 26)
    p2, l2, _, _, _, ck2, ss2, _ = setup_sft(cfg2, None, ds, None, model_cfg=_mc())
    assert ss2["total_steps"] == 25 and torch.equal(p2.flat.flat, policy.flat.flat)
    assert torch.equal(p2.optimizer.m, policy.optimizer.m)
    assert l2.state_dict() == {"epoch": 1, "pos": (25 - 16) * 16}  # 25 batches of 16 over a 256-sample epoch


def test_dpo_and_rm_improve_accuracy(tmp_path):
    ds = RandomPreferenceDataset(256, 64, seed=0)
    cfg = _cfg(tmp_path / "dpo", "dpo", 20, reference_policy_kl_penalty=0.5)
    policy, loader, vl, loss_fn, logger, ck, ss, cfg = setup_dpo(cfg, None, ds, None, model_cfg=_mc())
    hist = []
    dpo_train(policy, loader, vl, None, loss_fn, logger, ck, ss, cfg, step_callback=lambda s, m: hist.append(m["train"]))
    assert hist[0]["accuracy"] <= 0.6 and hist[-1]["accuracy"] > 0.8, [h["accuracy"] for h in hist]
    assert hist[-1]["loss"] < hist[0]["loss"]
    cfg = _cfg(tmp_path / "rm", "rm", 30)
    policy, loader, vl, loss_fn, logger, ck, ss, cfg = setup_rm(cfg, None, ds, None, model_cfg=_mc())
    hist = []
    rm_train(policy, loader, vl, None, loss_fn, logger, ck, ss, cfg, step_callback=lambda s, m: hist.append(m["train"]))
    acc = [h["accuracy"] for h in hist]
    assert sum(acc[-5:]) > sum(acc[:5]) and hist[-1]["loss"] < hist[0]["loss"], acc
