"""PPO with a learned critic: rollouts -> rewards -> value inference -> GAE (optionally VAPO's decoupled /
length-adaptive lambda) -> clipped policy update -> clipped value regression.

Step phases follow nemo_rl/algorithms/ppo.py:1318-1702. The critic is a second :class:`PolicyWorker` whose model has a
scalar head (``value_head=True``); both models live on every rank (SPMD) and shard their optimizer state the same way.
"""

from __future__ import annotations

from typing import Callable, Optional

import torch

from rl_b200.algorithms.advantage_estimator import GAEAdvantageEstimator
from rl_b200.algorithms.grpo import (GRPO_DEFAULTS, _aggregate_train_metrics, compute_and_apply_seq_logprob_error_masking, _all_reduce_scalars, _is_main, _ShardedPromptLoader, _world,
                                     build_train_data, refit_policy_generation, save_checkpoint)
from rl_b200.algorithms.loss.loss_functions import ClippedPGLossFn, MseValueLossFn
from rl_b200.algorithms.reward_functions import apply_reward_shaping, scale_rewards
from rl_b200.algorithms.utils import compute_performance_metrics, set_seed
from rl_b200.data.llm_message_utils import batched_message_log_to_flat_message
from rl_b200.experience.rollouts import run_multi_turn_rollout
from rl_b200.utils.checkpoint import CheckpointManager
from rl_b200.utils.logger import Logger
from rl_b200.utils.timer import Timer

PPO_DEFAULTS = dict(
    num_prompts_per_step=32, num_generations_per_prompt=1, max_num_epochs=1, max_num_steps=1_000_000, max_rollout_turns=1,
    val_period=0, seed=42, gamma=1.0, gae_lambda=0.95, lambda_critic=None, length_adaptive_alpha=None,
    normalize_advantages=True, value_clip=0.2, num_value_warmup_steps=0, policy_epochs=1, value_epochs=1,
    reward_shaping=None, reward_scaling=None,
    # names of the reference's PPOConfig (nemo_rl/algorithms/ppo.py:168-216) that map onto the ones above or add behaviour
    ppo_epochs=None,                    # passes over the batch for the policy AND the critic (overrides policy_epochs / value_epochs)
    policy_training_start_step=None,    # the critic trains alone before this step (overrides num_value_warmup_steps)
    overlong_filtering=False,           # truncated samples do not contribute to either loss
    seq_logprob_error_threshold=None,   # sequences whose trainer / engine log-probabilities disagree by more are masked
    val_at_start=False, val_at_end=False, val_batch_size=256,
)


def setup(cfg: dict, tokenizer, dataset, val_dataset, task_to_env, model_cfg=None, value_model_cfg=None):
    """Returns (policy, value, generation, loader, policy_loss, value_loss, logger, checkpointer, save_state, cfg)."""
    import copy

    from rl_b200.data.collate import rl_collate_fn
    from rl_b200.policy.worker import PolicyWorker

    from rl_b200.policy.worker import ensure_parallel

    ensure_parallel(cfg["policy"])
    rank, world = _world()
    p = dict(PPO_DEFAULTS)
    p.update(cfg.get("ppo") or {})
    if p.get("ppo_epochs"):
        p["policy_epochs"] = p["value_epochs"] = int(p["ppo_epochs"])
    if p.get("policy_training_start_step") is not None:
        p["num_value_warmup_steps"] = int(p["policy_training_start_step"])
    cfg["ppo"] = p
    set_seed(p["seed"] + rank)
    logger = Logger(cfg.get("logger"), is_main=_is_main())
    checkpointer = CheckpointManager(cfg.get("checkpointing"))
    save_state = {"current_step": 0, "total_steps": 0, "current_epoch": 0, "consumed_samples": 0, "total_valid_tokens": 0, "val_reward": -1e9}
    loader = _ShardedPromptLoader(dataset, p["num_prompts_per_step"], rl_collate_fn, bool((cfg.get("data") or {}).get("shuffle", True)),
                                  p["seed"], rank, world)
    loss_cfg = dict(cfg.get("loss_fn") or {})
    needs_ref = loss_cfg.get("reference_policy_kl_penalty", 0.0) != 0
    loss_cfg.setdefault("reference_policy_kl_penalty", 0.0)
    policy = PolicyWorker(cfg["policy"], model_cfg=model_cfg, tokenizer=tokenizer, init_reference_model=needs_ref, seed=p["seed"])
    vcfg = dict(cfg.get("value") or cfg["policy"])
    vm = copy.deepcopy(value_model_cfg or model_cfg)
    if vm is not None:
        vm.value_head = True
    value = PolicyWorker(vcfg, model_cfg=vm, tokenizer=tokenizer, init_reference_model=False, seed=p["seed"] + 1)
    generation = policy.build_generation(cfg["policy"].get("generation"))
    return (policy, value, generation, loader, ClippedPGLossFn(loss_cfg), MseValueLossFn({"value_clip": p["value_clip"]}), logger,
            checkpointer, save_state, cfg)


def ppo_train(policy, value, generation, loader, tokenizer, policy_loss, value_loss, task_to_env, logger, checkpointer, save_state,
              cfg, step_callback: Optional[Callable] = None) -> dict:
    rank, world = _world()
    p, pcfg = cfg["ppo"], cfg["policy"]
    timer = Timer()
    pad = tokenizer.pad_token_id if tokenizer is not None and tokenizer.pad_token_id is not None else 0
    gae = GAEAdvantageEstimator({"gamma": p["gamma"], "lambda": p["gae_lambda"], "lambda_critic": p["lambda_critic"] or p["gae_lambda"],
                                 "length_adaptive_alpha": p["length_adaptive_alpha"], "normalize_advantages": p["normalize_advantages"]})
    n_gen = p["num_generations_per_prompt"]
    use_ref = policy_loss.cfg["reference_policy_kl_penalty"] != 0
    total_steps, epoch = save_state["total_steps"], save_state["current_epoch"]
    last: dict = {}
    while epoch < p["max_num_epochs"] and total_steps < p["max_num_steps"]:
        for batch in loader:
            if total_steps >= p["max_num_steps"]:
                break
            with timer.time("total_step_time"):
                repeated = batch.repeat_interleave(n_gen)
                repeated["message_log"] = [[dict(m) for m in log] for log in repeated["message_log"]]
                repeated["rng_ids"] = repeated["idx"] * n_gen + torch.arange(n_gen).repeat(batch.size)
                prompt_flat, _ = batched_message_log_to_flat_message(repeated["message_log"], {"token_ids": pad})
                with timer.time("prepare_for_generation/total"):
                    refit_policy_generation(policy, generation, timer)
                with timer.time("generation"):
                    repeated, rollout_metrics = run_multi_turn_rollout(generation, repeated, tokenizer, task_to_env,
                                                                       pcfg["max_total_sequence_length"], p["max_rollout_turns"], pad_token_id=pad)
                    generation.finish_generation()
                repeated = scale_rewards(repeated, p.get("reward_scaling"))
                repeated = apply_reward_shaping(repeated, p.get("reward_shaping"))
                rewards = repeated["total_reward"].float()
                if p.get("overlong_filtering"):
                    repeated["loss_multiplier"] = repeated["loss_multiplier"] * (~repeated["truncated"].bool()).float()
                train_data = build_train_data(repeated, pad)
                with timer.time("policy_and_reference_logprobs"):
                    policy.prepare_for_lp_inference()
                    train_data["prev_logprobs"] = policy.get_logprobs(train_data)["logprobs"]
                    train_data["reference_policy_logprobs"] = (policy.get_reference_policy_logprobs(train_data)["reference_logprobs"]
                                                               if use_ref else torch.zeros_like(train_data["prev_logprobs"]))
                mask_metrics = compute_and_apply_seq_logprob_error_masking(train_data, p.get("seq_logprob_error_threshold"))
                with timer.time("value_inference"):
                    old_values = value.score(train_data)["values"]
                with timer.time("advantage_calculation"):
                    adv, returns = gae.compute_advantage(prompt_flat["token_ids"], rewards, train_data["token_mask"], values=old_values)
                    train_data["advantages"], train_data["returns"], train_data["old_values"] = adv, returns, old_values
                res = None
                if total_steps >= p["num_value_warmup_steps"]:
                    with timer.time("policy_training"):
                        policy.prepare_for_training()
                        for _ in range(p["policy_epochs"]):
                            res = policy.train(train_data, policy_loss, gbs=pcfg["train_global_batch_size"], mbs=pcfg["train_micro_batch_size"])
                with timer.time("value_training"):
                    value.prepare_for_training()
                    for _ in range(p["value_epochs"]):
                        vres = value.train(train_data, value_loss, gbs=pcfg["train_global_batch_size"], mbs=pcfg["train_micro_batch_size"])
            total_steps += 1
            metrics = _aggregate_train_metrics(res) if res is not None else {}
            metrics.update(mask_metrics)
            vmetrics = _aggregate_train_metrics(vres)
            metrics.update({f"value_{k}": v for k, v in vmetrics.items() if k in ("loss", "grad_norm", "value_mean", "value_clip_frac")})
            counts = _all_reduce_scalars({"r": float(rewards.sum()), "n": float(rewards.numel()), "tok": float(train_data["input_lengths"].sum()),
                                          "gen": float(repeated["generation_lengths"].sum())})
            metrics["reward"] = counts["r"] / max(1.0, counts["n"])
            save_state.update(current_step=total_steps, total_steps=total_steps, current_epoch=epoch)
            timing = timer.get_timing_metrics("sum")
            perf = compute_performance_metrics(timing, num_gpus=world, total_tokens=int(counts["tok"]), generated_tokens=int(counts["gen"]))
            ck = cfg.get("checkpointing") or {}
            if checkpointer.enabled and ck.get("save_period") and total_steps % ck["save_period"] == 0:
                save_checkpoint(policy, loader, checkpointer, save_state, cfg, total_steps)
            if logger is not None:
                logger.log_metrics(metrics, total_steps, prefix="train")
                logger.log_metrics(timing, total_steps, prefix="timing/train")
                logger.log_metrics(perf, total_steps, prefix="performance")
            if _is_main():
                print(f"[ppo] step {total_steps}: reward={metrics['reward']:.4f} policy_loss={metrics.get('loss', float('nan')):.5f} "
                      f"value_loss={metrics.get('value_loss', float('nan')):.5f} step_time={timing.get('total_step_time', 0):.2f}s", flush=True)
            last = {"train": metrics, "timing": timing, "performance": perf}
            if step_callback is not None:
                step_callback(total_steps, last)
            timer.reset()
        epoch += 1
        save_state["current_epoch"] = epoch
    return last


def async_ppo_train(policy, value, generation, loader, tokenizer, policy_loss, value_loss, task_to_env, logger, checkpointer, save_state,
                    cfg, step_callback: Optional[Callable] = None, buffer=None) -> dict:
    """Off-policy PPO: rollouts run ahead of training by up to ``ppo.async_ppo.max_trajectory_age_steps`` weight versions (the
    replay buffer and staleness rules of :mod:`rl_b200.algorithms.async_grpo`); values and GAE are computed with the critic
    that is current when a trajectory is trained on, and the policy loss corrects for the stale sampler through its
    importance-sampling term. Counterpart of ``async_ppo_train`` (nemo_rl/algorithms/ppo.py:2062)."""
    from rl_b200.algorithms.async_grpo import ReplayBuffer

    p, pcfg = cfg["ppo"], cfg["policy"]
    a = dict(max_trajectory_age_steps=1)
    a.update(p.get("async_ppo") or {})
    max_age = int(a["max_trajectory_age_steps"])
    assert policy_loss.cfg["use_importance_sampling_correction"] or max_age == 0, \
        "off-policy trajectories need loss_fn.use_importance_sampling_correction=true"
    timer = Timer()
    pad = tokenizer.pad_token_id if tokenizer is not None and tokenizer.pad_token_id is not None else 0
    gae = GAEAdvantageEstimator({"gamma": p["gamma"], "lambda": p["gae_lambda"], "lambda_critic": p["lambda_critic"] or p["gae_lambda"],
                                 "length_adaptive_alpha": p["length_adaptive_alpha"], "normalize_advantages": p["normalize_advantages"]})
    n_gen = p["num_generations_per_prompt"]
    use_ref = policy_loss.cfg["reference_policy_kl_penalty"] != 0
    buffer = buffer if buffer is not None else ReplayBuffer(max_size=4 * (max_age + 1))
    version = save_state.get("weight_version", 0)
    total_steps = save_state["total_steps"]
    it = iter(loader)
    next_target, exhausted, last = total_steps, False, {}
    while total_steps < p["max_num_steps"]:
        with timer.time("total_step_time"):
            refit_policy_generation(policy, generation, timer)
            while not exhausted and next_target <= total_steps + max_age and len(buffer) < buffer.max_size:
                try:
                    batch = next(it)
                except StopIteration:
                    exhausted = True
                    break
                repeated = batch.repeat_interleave(n_gen)
                repeated["message_log"] = [[dict(m) for m in log] for log in repeated["message_log"]]
                repeated["rng_ids"] = repeated["idx"] * n_gen + torch.arange(n_gen).repeat(batch.size)
                pf, _ = batched_message_log_to_flat_message(repeated["message_log"], {"token_ids": pad})
                repeated["_prompt_ids"] = pf["token_ids"]
                with timer.time("generation"):
                    repeated, _ = run_multi_turn_rollout(generation, repeated, tokenizer, task_to_env, pcfg["max_total_sequence_length"],
                                                         p["max_rollout_turns"], pad_token_id=pad)
                buffer.push(repeated, version, next_target)
                next_target += 1
            generation.finish_generation()
            item = buffer.sample(version, max_age)
            if item is None:
                break
            repeated = apply_reward_shaping(scale_rewards(item["batch"], p.get("reward_scaling")), p.get("reward_shaping"))
            rewards = repeated["total_reward"].float()
            train_data = build_train_data(repeated, pad)
            policy.prepare_for_lp_inference()
            train_data["prev_logprobs"] = policy.get_logprobs(train_data)["logprobs"]
            train_data["reference_policy_logprobs"] = (policy.get_reference_policy_logprobs(train_data)["reference_logprobs"]
                                                       if use_ref else torch.zeros_like(train_data["prev_logprobs"]))
            old_values = value.score(train_data)["values"]
            adv, returns = gae.compute_advantage(repeated["_prompt_ids"], rewards, train_data["token_mask"], values=old_values)
            train_data["advantages"], train_data["returns"], train_data["old_values"] = adv, returns, old_values
            res = None
            if total_steps >= p["num_value_warmup_steps"]:
                policy.prepare_for_training()
                res = policy.train(train_data, policy_loss, gbs=pcfg["train_global_batch_size"], mbs=pcfg["train_micro_batch_size"])
                version += 1
            value.prepare_for_training()
            vres = value.train(train_data, value_loss, gbs=pcfg["train_global_batch_size"], mbs=pcfg["train_micro_batch_size"])
        total_steps += 1
        metrics = _aggregate_train_metrics(res) if res is not None else {}
        metrics.update({f"value_{k}": v for k, v in _aggregate_train_metrics(vres).items() if k in ("loss", "grad_norm")})
        c = _all_reduce_scalars({"r": float(rewards.sum()), "n": float(rewards.numel())})
        metrics.update(reward=c["r"] / max(1.0, c["n"]), trajectory_age=float(item["age"]), buffer_size=float(len(buffer)))
        save_state.update(current_step=total_steps, total_steps=total_steps, weight_version=version)
        if logger is not None:
            logger.log_metrics(metrics, total_steps, prefix="train")
        if _is_main():
            print(f"[async_ppo] step {total_steps}: reward={metrics['reward']:.4f} value_loss={metrics.get('value_loss', float('nan')):.5f} "
                  f"age={item['age']} buffer={len(buffer)}", flush=True)
        last = {"train": metrics, "timing": timer.get_timing_metrics("sum")}
        if step_callback is not None:
            step_callback(total_steps, last)
        timer.reset()
    return last
