"""On-policy distillation: the student generates, the teacher scores the student's own sequences with its top-k
logits, and the student minimises a (forward / reverse / mixed) KL to the teacher on those positions.

Phases follow nemo_rl/algorithms/distillation.py:776-939: rollout -> teacher ``get_topk_logits`` -> student training
with :class:`DistillationLossFn`. The teacher is a frozen :class:`PolicyWorker` (no optimizer, no reference copy).
"""

from __future__ import annotations

from typing import Callable, Optional

import torch

from rl_b200.algorithms.grpo import (_aggregate_train_metrics, _all_reduce_scalars, _ShardedPromptLoader, _is_main, _world, build_train_data,
                                     refit_policy_generation, save_checkpoint, validate)
from rl_b200.algorithms.loss.loss_functions import DistillationLossFn
from rl_b200.algorithms.utils import set_seed
from rl_b200.experience.rollouts import run_multi_turn_rollout
from rl_b200.utils.checkpoint import CheckpointManager
from rl_b200.utils.logger import Logger
from rl_b200.utils.timer import Timer

DISTILLATION_DEFAULTS = dict(num_prompts_per_step=32, num_generations_per_prompt=1, max_num_epochs=1, max_num_steps=1_000_000,
                             max_rollout_turns=1, topk_logits_k=64, seed=42, val_period=0, val_batch_size=64, val_at_start=False,
                             val_at_end=False, max_val_samples=512, val_num_generations_per_prompt=1)


def setup(cfg: dict, tokenizer, dataset, val_dataset, task_to_env, student_cfg=None, teacher_cfg=None, teacher=None):
    from rl_b200.data.collate import rl_collate_fn
    from rl_b200.policy.worker import PolicyWorker

    from rl_b200.policy.worker import ensure_parallel

    ensure_parallel(cfg["policy"])
    rank, world = _world()
    d = dict(DISTILLATION_DEFAULTS)
    d.update(cfg.get("distillation") or {})
    cfg["distillation"] = d
    set_seed(d["seed"] + rank)
    logger = Logger(cfg.get("logger"), is_main=_is_main())
    checkpointer = CheckpointManager(cfg.get("checkpointing"))
    save_state = {"current_step": 0, "total_steps": 0, "current_epoch": 0, "val_reward": -1e9, "consumed_samples": 0, "total_valid_tokens": 0}
    resume = checkpointer.get_resume_paths() if checkpointer.enabled else None
    if resume:
        save_state.update(checkpointer.load_training_info(resume["root"]) or {})
    loader = _ShardedPromptLoader(dataset, d["num_prompts_per_step"], rl_collate_fn, bool((cfg.get("data") or {}).get("shuffle", True)),
                                  d["seed"], rank, world)
    if resume and resume.get("dataloader"):
        loader.load_state_dict(torch.load(resume["dataloader"], weights_only=False))
    student = PolicyWorker(cfg["policy"], model_cfg=student_cfg, tokenizer=tokenizer, init_reference_model=False, seed=d["seed"])
    if resume and resume.get("weights"):
        student.load_checkpoint(resume["weights"], resume.get("optimizer"))
    # validation prompts (the student's accuracy on held-out tasks is the number distillation is judged by)
    loader.val_loader = None      # (rides on the training loader: the tuple this function returns is part of the entrypoints' contract)
    if val_dataset is not None and len(val_dataset):
        vb = max(world, (min(d["val_batch_size"], len(val_dataset)) // world) * world)
        loader.val_loader = _ShardedPromptLoader(val_dataset, vb, rl_collate_fn, False, 0, rank, world)
    if teacher is None:
        teacher = PolicyWorker(cfg.get("teacher") or cfg["policy"], model_cfg=teacher_cfg, tokenizer=tokenizer, init_optimizer=False,
                               init_reference_model=False, seed=d["seed"] + 17)
    generation = student.build_generation(cfg["policy"].get("generation"))
    loss_fn = DistillationLossFn(cfg.get("loss_fn"))
    return student, teacher, generation, loader, loss_fn, logger, checkpointer, save_state, cfg


def distillation_train(student, teacher, generation, loader, tokenizer, loss_fn, task_to_env, logger, checkpointer, save_state, cfg,
                       step_callback: Optional[Callable] = None) -> dict:
    rank, world = _world()
    d, pcfg = cfg["distillation"], cfg["policy"]
    timer = Timer()
    pad = tokenizer.pad_token_id if tokenizer is not None and tokenizer.pad_token_id is not None else 0
    n_gen = d["num_generations_per_prompt"]
    total_steps, epoch = save_state["total_steps"], save_state["current_epoch"]
    last: dict = {}
    val_loader = getattr(loader, "val_loader", None)
    # the validation routine is GRPO's (rollouts on held-out prompts, mean reward): give it the keys it reads
    vcfg = dict(cfg, grpo=dict(val_num_generations_per_prompt=d["val_num_generations_per_prompt"], max_rollout_turns=d["max_rollout_turns"],
                               max_val_samples=d["max_val_samples"] or 1 << 30))
    if val_loader is not None and d["val_at_start"] and total_steps == 0:
        val, _ = validate(student, generation, val_loader, tokenizer, task_to_env, 0, vcfg, logger)
        save_state["val_reward"] = val.get("accuracy", -1e9)
    while epoch < d["max_num_epochs"] and total_steps < d["max_num_steps"]:
        for batch in loader:
            if total_steps >= d["max_num_steps"]:
                break
            with timer.time("total_step_time"):
                repeated = batch.repeat_interleave(n_gen)
                repeated["message_log"] = [[dict(m) for m in log] for log in repeated["message_log"]]
                repeated["rng_ids"] = repeated["idx"] * n_gen + torch.arange(n_gen).repeat(batch.size)
                with timer.time("prepare_for_generation/total"):
                    refit_policy_generation(student, generation, timer)
                with timer.time("generation"):
                    repeated, rollout_metrics = run_multi_turn_rollout(generation, repeated, tokenizer, task_to_env,
                                                                       pcfg["max_total_sequence_length"], d["max_rollout_turns"], pad_token_id=pad)
                    generation.finish_generation()
                train_data = build_train_data(repeated, pad)
                with timer.time("teacher_logprob_inference"):
                    topk = teacher.get_topk_logits(train_data, d["topk_logits_k"])
                    train_data["teacher_topk_logits"] = topk["topk_logits"]
                    train_data["teacher_topk_indices"] = topk["topk_indices"]
                with timer.time("policy_training"):
                    student.prepare_for_training()
                    res = student.train(train_data, loss_fn, gbs=pcfg["train_global_batch_size"], mbs=pcfg["train_micro_batch_size"])
            total_steps += 1
            metrics = _aggregate_train_metrics(res)
            metrics.update({k: v for k, v in rollout_metrics.items() if isinstance(v, (int, float))})
            is_last = total_steps >= d["max_num_steps"]
            if val_loader is not None and ((d["val_period"] > 0 and total_steps % d["val_period"] == 0) or (is_last and d["val_at_end"])):
                val, _ = validate(student, generation, val_loader, tokenizer, task_to_env, total_steps, vcfg, logger)
                save_state["val_reward"] = val.get("accuracy", save_state["val_reward"])
                metrics["val_accuracy"] = save_state["val_reward"]
            save_state.update(current_step=total_steps, total_steps=total_steps, current_epoch=epoch,
                              consumed_samples=save_state["consumed_samples"] + repeated.size * world,
                              total_valid_tokens=save_state["total_valid_tokens"] + int(train_data["token_mask"].sum()) * world)
            timing = timer.get_timing_metrics("sum")
            ck = cfg.get("checkpointing") or {}
            if checkpointer.enabled and ck.get("save_period") and total_steps % ck["save_period"] == 0:
                save_checkpoint(student, loader, checkpointer, save_state, cfg, total_steps)
            if logger is not None:
                logger.log_metrics(metrics, total_steps, prefix="train")
                logger.log_metrics(timing, total_steps, prefix="timing/train")
            if _is_main():
                print(f"[distillation] step {total_steps}: loss={metrics['loss']:.5f} step_time={timing.get('total_step_time', 0):.2f}s", flush=True)
            last = {"train": metrics, "timing": timing}
            if step_callback is not None:
                step_callback(total_steps, last)
            timer.reset()
        epoch += 1
        save_state["current_epoch"] = epoch
    return last
