"""Off-policy ("k-step-off") GRPO: a replay buffer of trajectories tagged with the weight version that generated
them, an age bound on what may be trained on, and importance-sampling correction in the loss.

Semantics follow nemo_rl/algorithms/grpo.py:4074-5462 and async_utils/replay_buffer.py:40: trajectories are produced
for a *target* training step, at most ``max_trajectory_age_steps`` versions behind the weights that train on them;
samples older than that are dropped; the buffer state is checkpointable. This module is the COLOCATED form: generation
and training share the GPUs, so collection runs ahead in bursts between optimizer steps; the data path, staleness
accounting and loss are those of the split form. With ``policy.generation.colocated.enabled: false`` the job is split into
training and generation ranks that run at the same time: ``rl_b200/algorithms/noncolocated.py``.
"""

from __future__ import annotations

import collections
from typing import Callable, Optional

import torch

from rl_b200.algorithms.advantage_estimator import create_advantage_estimator
from rl_b200.algorithms.grpo import (_aggregate_train_metrics, _all_reduce_scalars, _is_main, _world, build_train_data, refit_policy_generation,
                                     save_checkpoint)
from rl_b200.algorithms.utils import calculate_baseline_and_std_per_prompt
from rl_b200.data.llm_message_utils import batched_message_log_to_flat_message
from rl_b200.distributed.batched_data_dict import BatchedDataDict
from rl_b200.experience.rollouts import run_multi_turn_rollout
from rl_b200.utils.timer import Timer

ASYNC_DEFAULTS = dict(enabled=True, max_trajectory_age_steps=1, max_generation_failures=0, in_flight_weight_updates=False,
                      recompute_kv_cache_after_weight_updates=False)


class ReplayBuffer:
    """FIFO of (trajectory batch, generation weight version, target step) with age-bounded sampling."""

    def __init__(self, max_size: int = 64):
        self.items: collections.deque = collections.deque()
        self.max_size = max_size
        self.dropped_stale = 0

    def __len__(self):
        return len(self.items)

    def push(self, batch: BatchedDataDict, weight_version: int, target_step: int) -> bool:
        if len(self.items) >= self.max_size:
            return False
        self.items.append({"batch": batch, "weight_version": weight_version, "target_step": target_step})
        return True

    def sample(self, current_version: int, max_age: int) -> Optional[dict]:
        """Oldest trajectory that is at most ``max_age`` versions behind ``current_version``; staler ones are dropped."""
        while self.items:
            it = self.items[0]
            age = current_version - it["weight_version"]
            if age > max_age:
                self.items.popleft()
                self.dropped_stale += 1
                continue
            self.items.popleft()
            it["age"] = age
            return it
        return None

    def state_dict(self) -> dict:
        return {"items": list(self.items), "dropped_stale": self.dropped_stale}

    def load_state_dict(self, sd: dict) -> None:
        self.items = collections.deque(sd["items"])
        self.dropped_stale = sd.get("dropped_stale", 0)


def _collect(policy, generation, batch, tokenizer, task_to_env, cfg, pad, timer) -> tuple[BatchedDataDict, dict]:
    g, pcfg = cfg["grpo"], cfg["policy"]
    n_gen = g["num_generations_per_prompt"]
    repeated = batch.repeat_interleave(n_gen)
    repeated["message_log"] = [[dict(m) for m in log] for log in repeated["message_log"]]
    repeated["rng_ids"] = repeated["idx"] * n_gen + torch.arange(n_gen).repeat(batch.size)
    pf, _ = batched_message_log_to_flat_message(repeated["message_log"], {"token_ids": pad})
    repeated["_prompt_ids"] = pf["token_ids"]
    with timer.time("generation"):
        repeated, m = run_multi_turn_rollout(generation, repeated, tokenizer, task_to_env, pcfg["max_total_sequence_length"],
                                             g["max_rollout_turns"], pad_token_id=pad)
    return repeated, m


def async_grpo_train(policy, generation, dataloader, tokenizer, loss_fn, task_to_env, logger, checkpointer, save_state, cfg,
                     step_callback: Optional[Callable] = None, buffer: Optional[ReplayBuffer] = None) -> dict:
    rank, world = _world()
    g, pcfg = cfg["grpo"], cfg["policy"]
    a = dict(ASYNC_DEFAULTS)
    a.update(g.get("async_grpo") or {})
    max_age = int(a["max_trajectory_age_steps"])
    assert loss_fn.cfg["use_importance_sampling_correction"] or max_age == 0, \
        "off-policy trajectories need loss_fn.use_importance_sampling_correction=true"
    timer = Timer()
    pad = tokenizer.pad_token_id if tokenizer is not None and tokenizer.pad_token_id is not None else 0
    adv_estimator = create_advantage_estimator(g, cfg.get("loss_fn") or {})
    buffer = buffer if buffer is not None else ReplayBuffer(max_size=4 * (max_age + 1))
    ck = cfg.get("checkpointing") or {}
    resume = checkpointer.get_resume_paths() if (checkpointer is not None and checkpointer.enabled) else None
    if resume and resume.get("replay_buffer") and len(buffer) == 0:
        # trajectories that were collected but not yet trained on survive a restart (their age is still checked on sampling)
        path = resume["replay_buffer"] if rank == 0 else f"{resume['replay_buffer']}.rank{rank}"
        import os

        if os.path.exists(path):
            buffer.load_state_dict(torch.load(path, weights_only=False))
    use_ref = loss_fn.cfg["reference_policy_kl_penalty"] != 0 and policy.ref_flat is not None
    version = save_state.get("weight_version", 0)
    total_steps = save_state["total_steps"]
    data_iter = iter(dataloader)
    next_target = total_steps
    last: dict = {}
    exhausted = False
    while total_steps < g["max_num_steps"]:
        with timer.time("total_step_time"):
            # collection runs ahead: trajectories for steps [total_steps, total_steps + max_age] come from the current weights
            refit_policy_generation(policy, generation, timer)
            while not exhausted and next_target <= total_steps + max_age and len(buffer) < buffer.max_size:
                try:
                    batch = next(data_iter)
                except StopIteration:
                    exhausted = True
                    break
                traj, _ = _collect(policy, generation, batch, tokenizer, task_to_env, cfg, pad, timer)
                buffer.push(traj, version, next_target)
                next_target += 1
            generation.finish_generation()
            item = buffer.sample(version, max_age)
            if item is None:
                break
            repeated = item["batch"]
            rewards = repeated["total_reward"].float()
            train_data = build_train_data(repeated, pad)
            train_data["rewards"] = rewards
            with timer.time("policy_and_reference_logprobs"):
                policy.prepare_for_lp_inference()
                train_data["prev_logprobs"] = policy.get_logprobs(train_data)["logprobs"]
                train_data["reference_policy_logprobs"] = (policy.get_reference_policy_logprobs(train_data)["reference_logprobs"]
                                                           if use_ref else torch.zeros_like(train_data["prev_logprobs"]))
            train_data["advantages"] = adv_estimator.compute_advantage(repeated["_prompt_ids"], rewards, train_data["token_mask"],
                                                                       valid_mask=torch.ones_like(rewards))
            with timer.time("policy_training"):
                policy.prepare_for_training()
                res = policy.train(train_data, loss_fn, gbs=pcfg["train_global_batch_size"], mbs=pcfg["train_micro_batch_size"])
            version += 1
        total_steps += 1
        metrics = _aggregate_train_metrics(res)
        c = _all_reduce_scalars({"r": float(rewards.sum()), "n": float(rewards.numel())})
        metrics.update(reward=c["r"] / max(1.0, c["n"]), trajectory_age=float(item["age"]), buffer_size=float(len(buffer)),
                       dropped_stale=float(buffer.dropped_stale))
        save_state.update(current_step=total_steps, total_steps=total_steps, weight_version=version)
        if checkpointer is not None and checkpointer.enabled and ck.get("save_period") and total_steps % ck["save_period"] == 0:
            save_checkpoint(policy, dataloader, checkpointer, save_state, cfg, total_steps, extra_files={"replay_buffer.pt": buffer.state_dict()})
        timing = timer.get_timing_metrics("sum")
        if logger is not None:
            logger.log_metrics(metrics, total_steps, prefix="train")
            logger.log_metrics(timing, total_steps, prefix="timing/train")
        if _is_main():
            print(f"[async_grpo] step {total_steps}: loss={metrics['loss']:.5f} reward={metrics['reward']:.4f} age={item['age']} "
                  f"buffer={len(buffer)}", flush=True)
        last = {"train": metrics, "timing": timing}
        if step_callback is not None:
            step_callback(total_steps, last)
        timer.reset()
    return last
