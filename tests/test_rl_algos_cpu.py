"""PPO, on-policy distillation and off-policy (async) GRPO loops on CPU with tiny models."""

import pytest
import torch

from rl_b200.algorithms import async_grpo, distillation, grpo, ppo
from rl_b200.data.datasets.synthetic import RandomTokenPromptDataset
from rl_b200.environments.synthetic import TokenFractionEnv
from rl_b200.models.config import ModelConfig


def _mc():
    return ModelConfig(vocab_size=32, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=8, torch_dtype="float32")


def _policy_cfg(lr=5e-3):
    return dict(precision="float32", train_global_batch_size=16, train_micro_batch_size=8, logprob_batch_size=16,
                max_total_sequence_length=48, max_grad_norm=1.0, optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=lr, weight_decay=0.0)),
                generation=dict(max_new_tokens=8, temperature=1.0, stop_token_ids=[], kv_cache_tokens=4096, block_size=8, max_running=32))


def test_ppo_runs_and_value_loss_falls(tmp_path):
    ds = RandomTokenPromptDataset(256, 4, 8, 32, seed=0)
    env = {"synthetic": TokenFractionEnv({"target_token_id": 7})}
    cfg = {"ppo": dict(num_prompts_per_step=16, num_generations_per_prompt=1, max_num_steps=6, seed=0), "loss_fn": {},
           "policy": _policy_cfg(), "logger": dict(log_dir=str(tmp_path)), "checkpointing": dict(enabled=False)}
    policy, value, gen, loader, pl, vl, logger, ck, ss, cfg = ppo.setup(cfg, None, ds, None, env, model_cfg=_mc())
    hist = []
    ppo.ppo_train(policy, value, gen, loader, None, pl, vl, env, logger, ck, ss, cfg, step_callback=lambda s, m: hist.append(m["train"]))
    assert len(hist) == 6 and all(torch.isfinite(torch.tensor(h["value_loss"])) for h in hist)
    assert hist[-1]["value_loss"] <= hist[0]["value_loss"] + 1e-3


def test_distillation_validates_counts_and_resumes(tmp_path):
    """Validation on held-out prompts at start / every period / at the end, consumed-sample and token counters, and a resume
    from the last checkpoint that continues the step count with the student's weights."""
    ds = RandomTokenPromptDataset(256, 4, 8, 32, seed=0)
    val = RandomTokenPromptDataset(16, 4, 8, 32, seed=1)
    env = {"synthetic": TokenFractionEnv({"target_token_id": 7})}

    def cfg_(steps):
        return {"distillation": dict(num_prompts_per_step=8, max_num_steps=steps, topk_logits_k=8, seed=0, val_period=2, val_at_start=True,
                                     val_at_end=True, val_batch_size=8, max_val_samples=16),
                "loss_fn": dict(kl_type="forward"), "policy": _policy_cfg(1e-2), "logger": dict(log_dir=str(tmp_path / "logs")),
                "checkpointing": dict(enabled=True, checkpoint_dir=str(tmp_path / "ckpt"), save_period=2, keep_top_k=None)}

    student, teacher, gen, loader, loss_fn, logger, ck, ss, cfg = distillation.setup(cfg_(3), None, ds, val, env, student_cfg=_mc(), teacher_cfg=_mc())
    hist = []
    distillation.distillation_train(student, teacher, gen, loader, None, loss_fn, env, logger, ck, ss, cfg,
                                    step_callback=lambda s, m: hist.append(m["train"]))
    assert len(hist) == 3 and "val_accuracy" in hist[1] and "val_accuracy" in hist[2] and "val_accuracy" not in hist[0]
    assert ss["consumed_samples"] == 24 and ss["total_valid_tokens"] > 0 and ss["val_reward"] >= 0.0
    w = student.flat.flat.clone()
    # a new run finds step_2 and goes on from there
    student2, teacher2, gen2, loader2, loss_fn2, logger2, ck2, ss2, cfg2 = distillation.setup(cfg_(4), None, ds, val, env, student_cfg=_mc(),
                                                                                            teacher_cfg=_mc())
    assert ss2["total_steps"] == 2 and ss2["consumed_samples"] == 16 and not torch.equal(student2.flat.flat, w)
    steps = []
    distillation.distillation_train(student2, teacher2, gen2, loader2, None, loss_fn2, env, logger2, ck2, ss2, cfg2,
                                    step_callback=lambda s, m: steps.append(s))
    assert steps == [3, 4]


def test_ppo_reference_config_names(tmp_path):
    """``ppo_epochs`` / ``policy_training_start_step`` / ``overlong_filtering`` / ``seq_logprob_error_threshold`` of the reference's
    PPO config: the critic trains alone before the start step, truncated samples leave the losses, the masking metric is logged."""
    ds = RandomTokenPromptDataset(256, 4, 8, 32, seed=0)
    env = {"synthetic": TokenFractionEnv({"target_token_id": 7})}
    cfg = {"ppo": dict(num_prompts_per_step=8, num_generations_per_prompt=1, max_num_steps=3, seed=0, ppo_epochs=2, policy_training_start_step=2,
                       seq_logprob_error_threshold=10.0), "loss_fn": {},
           "policy": _policy_cfg(), "logger": dict(log_dir=str(tmp_path)), "checkpointing": dict(enabled=False)}
    policy, value, gen, loader, pl, vl, logger, ck, ss, cfg = ppo.setup(cfg, None, ds, None, env, model_cfg=_mc())
    assert cfg["ppo"]["policy_epochs"] == cfg["ppo"]["value_epochs"] == 2 and cfg["ppo"]["num_value_warmup_steps"] == 2
    w0 = policy.flat.flat.clone()
    hist = []

    def cb(step, m):
        hist.append(m["train"])
        if step == 2:      # two critic-only steps: the policy has not moved
            assert torch.equal(policy.flat.flat, w0)

    ppo.ppo_train(policy, value, gen, loader, None, pl, vl, env, logger, ck, ss, cfg, step_callback=cb)
    assert len(hist) == 3 and "loss" not in hist[0] and "loss" in hist[2] and not torch.equal(policy.flat.flat, w0)
    assert all("seq_logprob_error_masked_fraction" in h and h["seq_logprob_error_masked_fraction"] == 0.0 for h in hist)
    assert any(h["value_loss"] > 0.0 for h in hist)
    # every sample is cut by the 8-token limit (no stop token): with overlong filtering nothing is left to train on
    cfg2 = {"ppo": dict(num_prompts_per_step=8, num_generations_per_prompt=1, max_num_steps=1, seed=0, overlong_filtering=True), "loss_fn": {},
            "policy": _policy_cfg(), "logger": dict(log_dir=str(tmp_path)), "checkpointing": dict(enabled=False)}
    policy, value, gen, loader, pl, vl, logger, ck, ss, cfg2 = ppo.setup(cfg2, None, ds, None, env, model_cfg=_mc())
    out = ppo.ppo_train(policy, value, gen, loader, None, pl, vl, env, logger, ck, ss, cfg2)
    assert out["train"]["value_loss"] == 0.0 and out["train"]["loss"] == 0.0


def test_distillation_pulls_student_to_teacher(tmp_path):
    ds = RandomTokenPromptDataset(256, 4, 8, 32, seed=0)
    env = {"synthetic": TokenFractionEnv({})}
    cfg = {"distillation": dict(num_prompts_per_step=16, max_num_steps=12, topk_logits_k=8, seed=0), "loss_fn": dict(kl_type="forward"),
           "policy": _policy_cfg(1e-2), "logger": dict(log_dir=str(tmp_path)), "checkpointing": dict(enabled=False)}
    student, teacher, gen, loader, loss_fn, logger, ck, ss, cfg = distillation.setup(cfg, None, ds, None, env, student_cfg=_mc(), teacher_cfg=_mc())
    hist = []
    distillation.distillation_train(student, teacher, gen, loader, None, loss_fn, env, logger, ck, ss, cfg,
                                    step_callback=lambda s, m: hist.append(m["train"]["loss"]))
    assert hist[-1] < hist[0], hist


def test_async_grpo_ages_and_buffer(tmp_path):
    ds = RandomTokenPromptDataset(256, 4, 8, 32, seed=0)
    env = {"synthetic": TokenFractionEnv({"target_token_id": 7})}
    cfg = {"grpo": dict(num_prompts_per_step=4, num_generations_per_prompt=4, max_num_steps=5, val_period=0, seed=0,
                        async_grpo=dict(enabled=True, max_trajectory_age_steps=2)),
           "loss_fn": dict(use_importance_sampling_correction=True, reference_policy_kl_penalty=0.0),
           "policy": _policy_cfg(), "logger": dict(log_dir=str(tmp_path)), "checkpointing": dict(enabled=False)}
    policy, gen, loader, _, loss_fn, logger, ck, ss, cfg = grpo.setup(cfg, None, ds, None, env, model_cfg=_mc())
    hist = []
    async_grpo.async_grpo_train(policy, gen, loader, None, loss_fn, env, logger, ck, ss, cfg, step_callback=lambda s, m: hist.append(m["train"]))
    ages = [h["trajectory_age"] for h in hist]
    assert len(hist) == 5 and max(ages) <= 2 and max(ages) >= 1  # later steps train on stale trajectories
    buf = async_grpo.ReplayBuffer(4)
    for v in range(4):
        assert buf.push({"x": v}, v, v)
    assert not buf.push({"x": 9}, 9, 9)
    it = buf.sample(current_version=3, max_age=1)
    assert it["weight_version"] == 2 and buf.dropped_stale == 2
    b2 = async_grpo.ReplayBuffer(4)
    b2.load_state_dict(buf.state_dict())
    assert len(b2) == 1


def test_async_grpo_checkpoints_and_restores_its_replay_buffer(tmp_path):
    import os

    ds = RandomTokenPromptDataset(256, 4, 8, 32, seed=0)
    env = {"synthetic": TokenFractionEnv({"target_token_id": 7})}

    def cfg():
        return {"grpo": dict(num_prompts_per_step=4, num_generations_per_prompt=4, max_num_steps=2, val_period=0, seed=0,
                             async_grpo=dict(enabled=True, max_trajectory_age_steps=2)),
                "loss_fn": dict(use_importance_sampling_correction=True, reference_policy_kl_penalty=0.0),
                "policy": _policy_cfg(), "logger": dict(log_dir=str(tmp_path / "logs")),
                "checkpointing": dict(enabled=True, checkpoint_dir=str(tmp_path / "ck"), save_period=2, keep_top_k=2, metric_name=None)}

    policy, gen, loader, _, loss_fn, logger, ck, ss, c = grpo.setup(cfg(), None, ds, None, env, model_cfg=_mc())
    async_grpo.async_grpo_train(policy, gen, loader, None, loss_fn, env, logger, ck, ss, c)
    paths = ck.get_resume_paths()
    assert paths["replay_buffer"] and os.path.exists(paths["replay_buffer"])
    saved = torch.load(paths["replay_buffer"], weights_only=False)
    assert len(saved["items"]) >= 1                               # collected ahead of training, not yet consumed
    policy2, gen2, loader2, _, loss_fn2, logger2, ck2, ss2, c2 = grpo.setup(cfg(), None, ds, None, env, model_cfg=_mc())
    buf = async_grpo.ReplayBuffer(12)
    c2["grpo"]["max_num_steps"] = ss2["total_steps"]              # no further steps: only the restore path runs
    async_grpo.async_grpo_train(policy2, gen2, loader2, None, loss_fn2, env, logger2, ck2, ss2, c2, buffer=buf)
    assert len(buf) == len(saved["items"]) and ss2["total_steps"] == 2


def test_training_logprobs_follow_the_samplers_top_k_and_top_p(tmp_path):
    """Rollouts sampled with top-k / top-p: the trainer scores them under the same filtered distribution, so engine and
    trainer agree token by token; without the filters on the training side they would not."""
    ds = RandomTokenPromptDataset(64, 4, 8, 32, seed=0)
    env = {"synthetic": TokenFractionEnv({"target_token_id": 7})}
    pc = _policy_cfg()
    pc["generation"].update(top_k=6, top_p=0.8)
    cfg = {"grpo": dict(num_prompts_per_step=4, num_generations_per_prompt=4, max_num_steps=2, val_period=0, seed=0),
           "loss_fn": dict(reference_policy_kl_penalty=0.0), "policy": pc, "logger": dict(log_dir=str(tmp_path)), "checkpointing": dict(enabled=False)}
    policy, gen, loader, _, loss_fn, logger, ck, ss, cfg = grpo.setup(cfg, None, ds, None, env, model_cfg=_mc())
    assert policy.train_top_k == 6 and policy.train_top_p == 0.8
    hist = []
    grpo.grpo_train(policy, gen, loader, None, None, loss_fn, env, env, logger, ck, ss, cfg, step_callback=lambda s, m: hist.append(m["train"]))
    assert all(abs(h["token_mult_prob_error"] - 1.0) < 1e-3 for h in hist)
    policy.train_top_k, policy.train_top_p = None, 1.0          # unfiltered scoring of filtered samples: a visible gap
    hist2 = []
    cfg["grpo"].update(max_num_steps=3, max_num_epochs=5)
    grpo.grpo_train(policy, gen, loader, None, None, loss_fn, env, env, logger, ck, ss, cfg, step_callback=lambda s, m: hist2.append(m["train"]))
    assert hist2 and hist2[-1]["token_mult_prob_error"] > 1.05


def test_async_ppo_trains_on_stale_trajectories(tmp_path):
    ds = RandomTokenPromptDataset(256, 4, 8, 32, seed=0)
    env = {"synthetic": TokenFractionEnv({"target_token_id": 7})}
    cfg = {"ppo": dict(num_prompts_per_step=8, num_generations_per_prompt=1, max_num_steps=4, seed=0, async_ppo=dict(max_trajectory_age_steps=2)),
           "loss_fn": dict(use_importance_sampling_correction=True), "policy": _policy_cfg(), "logger": dict(log_dir=str(tmp_path)),
           "checkpointing": dict(enabled=False)}
    policy, value, gen, loader, pl, vl, logger, ck, ss, cfg = ppo.setup(cfg, None, ds, None, env, model_cfg=_mc())
    hist = []
    ppo.async_ppo_train(policy, value, gen, loader, None, pl, vl, env, logger, ck, ss, cfg, step_callback=lambda s, m: hist.append(m["train"]))
    assert len(hist) == 4 and max(h["trajectory_age"] for h in hist) >= 1 and max(h["trajectory_age"] for h in hist) <= 2
    assert all(torch.isfinite(torch.tensor(h["value_loss"])) for h in hist) and ss["weight_version"] == 4


def test_on_policy_distillation_routes_samples_to_teachers(tmp_path):
    """GRPO with the OPD estimator: two agent aliases share one teacher checkpoint (de-duplicated into one frozen worker), the
    advantage is teacher - student log-probability, and a student distilled from a teacher moves towards it."""
    from rl_b200.algorithms import grpo, opd
    from rl_b200.data.datasets.synthetic import RandomTokenPromptDataset
    from rl_b200.environments.synthetic import TokenFractionEnv
    from rl_b200.models.config import ModelConfig
    from rl_b200.policy.worker import PolicyWorker

    ocfg = dict(teacher_model_by_agent_name={"synthetic": "ckpt-A", "other": "ckpt-A", "third": "ckpt-B"}, default_teacher_alias="synthetic",
                non_colocated_teachers=dict(enabled=False, default_teacher_cfg=dict(micro_batch_size=4, some_override=1),
                                            teacher_overrides=dict(third=dict(precision="float32"))))
    tcs = opd.create_teacher_configs(ocfg)
    assert [t.alias for t in tcs] == ["synthetic", "third"] and tcs[0].micro_batch_size == 4 and tcs[0].overrides == {"some_override": 1}
    assert tcs[1].precision == "float32" and opd.alias_to_group_alias(ocfg) == {"synthetic": "synthetic", "other": "synthetic", "third": "third"}
    assert opd.resolve_teacher_aliases(["other", "nobody"], ocfg["teacher_model_by_agent_name"], "synthetic") == ["other", "synthetic"]
    with pytest.raises(KeyError):
        opd.resolve_teacher_aliases(["nobody"], ocfg["teacher_model_by_agent_name"], None)
    m = opd.teacher_routing_metrics(["synthetic", "other", "third"], ocfg["teacher_model_by_agent_name"])
    assert m["on_policy_distillation/teacher_alias_unique"] == 3 and m["on_policy_distillation/teacher_model_unique"] == 2

    mc = ModelConfig(vocab_size=32, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                     num_key_value_heads=2, head_dim=8, torch_dtype="float32")
    cfg = {"grpo": dict(num_prompts_per_step=4, num_generations_per_prompt=4, max_num_steps=40, val_period=0, seed=0,
                        adv_estimator=dict(name="opd", opd_coef=1.0)),
           "on_policy_distillation": dict(teacher_model_by_agent_name={"synthetic": "ckpt-A"}),
           "loss_fn": dict(reference_policy_kl_penalty=0.0),
           "policy": dict(precision="float32", train_global_batch_size=16, train_micro_batch_size=8, logprob_batch_size=16,
                          max_total_sequence_length=48, max_grad_norm=1.0,
                          optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=2e-2, weight_decay=0.0)),
                          generation=dict(max_new_tokens=8, temperature=1.0, stop_token_ids=[], kv_cache_tokens=4096, block_size=8, max_running=32)),
           "logger": dict(log_dir=str(tmp_path)), "checkpointing": dict(enabled=False)}
    ds = RandomTokenPromptDataset(256, 4, 8, 32, seed=0)
    env = {"synthetic": TokenFractionEnv({"target_token_id": 7})}
    policy, gen, loader, _, loss_fn, logger, ck, ss, cfg = grpo.setup(cfg, None, ds, None, env, model_cfg=mc)
    teacher = PolicyWorker(cfg["policy"], model_cfg=mc, init_optimizer=False, init_reference_model=False, seed=123)
    with torch.no_grad():   # a teacher with opinions: sharpen its output distribution
        teacher.model.output_weight.mul_(12.0)
    groups = ({"synthetic": opd.TeacherGroup(opd.TeacherConfig("synthetic", "ckpt-A"), cfg["policy"], worker=teacher)}, {"synthetic": "synthetic"})
    assert all(not p.requires_grad for p in teacher.model.parameters())
    hist = []
    grpo.grpo_train(policy, gen, loader, None, None, loss_fn, env, None, logger, ck, ss, cfg, step_callback=lambda s, m: hist.append(m["train"]),
                    teacher_groups=groups)
    gaps = [h["on_policy_distillation/teacher_student_logprob_gap_mean"] for h in hist]
    assert len(gaps) == 40 and gaps[0] < 0 and sum(gaps[-3:]) / 3 > sum(gaps[:3]) / 3 + 0.05, gaps     # the student closes in on the teacher
    assert hist[0]["on_policy_distillation/teacher_model_unique"] == 1.0
