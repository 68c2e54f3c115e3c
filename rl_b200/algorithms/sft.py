"""Supervised loops: SFT (teacher-forced NLL), DPO (preference optimisation against a frozen reference) and RM
(Bradley-Terry reward model). They share one driver: loader -> ``policy.train(batch, loss_fn)`` -> validation ->
checkpoint, following nemo_rl/algorithms/sft.py:379-680, dpo.py:526-821 and rm.py:469-747.

SPMD runtime: every rank takes its slice of each global batch; the loss functions normalise by global counts, so the
optimizer sees exactly the global-batch gradient.
"""

from __future__ import annotations

import os
from typing import Callable, Optional

import torch

from rl_b200.distributed.ft_launcher import beat as _ft_beat
import torch.distributed as dist

from rl_b200.algorithms.grpo import _ShardedPromptLoader, _aggregate_train_metrics, _agree_any, _all_reduce_scalars, _is_main, _world, save_checkpoint
from rl_b200.algorithms.loss.loss_functions import DPOLossFn, NLLLossFn, PreferenceLossFn
from rl_b200.algorithms.utils import set_seed
from rl_b200.distributed.batched_data_dict import BatchedDataDict
from rl_b200.utils.checkpoint import CheckpointManager
from rl_b200.utils.logger import Logger
from rl_b200.utils.timer import TimeoutChecker, Timer

SFT_DEFAULTS = dict(max_num_epochs=1, max_num_steps=1_000_000, val_period=10, val_batches=8, val_global_batch_size=32,
                    val_micro_batch_size=4, val_at_start=False, val_at_end=False, seed=42, only_unmask_final=False)
DPO_DEFAULTS = dict(SFT_DEFAULTS, reference_policy_kl_penalty=0.05, preference_average_log_probs=False,
                    sft_average_log_probs=False, preference_loss_weight=1.0, sft_loss_weight=0.0)
RM_DEFAULTS = dict(SFT_DEFAULTS)


def _setup_common(cfg: dict, key: str, defaults: dict, tokenizer, dataset, val_dataset, collate_fn: Callable, model_cfg=None,
                  needs_reference: bool = False, value_head: bool = False, policy=None):
    from rl_b200.policy.worker import PolicyWorker

    from rl_b200.policy.worker import ensure_parallel

    ensure_parallel(cfg["policy"])
    rank, world = _world()
    a = dict(defaults)
    a.update(cfg.get(key) or {})
    cfg[key] = a
    set_seed(a["seed"] + rank)
    logger = Logger(cfg.get("logger"), is_main=_is_main())
    checkpointer = CheckpointManager(cfg.get("checkpointing"))
    save_state = {"current_step": 0, "current_epoch": 0, "total_steps": 0, "consumed_samples": 0, "val_loss": None}
    resume = checkpointer.get_resume_paths() if checkpointer.enabled else None
    if resume:
        save_state.update(checkpointer.load_training_info(resume["root"]) or {})
    pcfg = cfg["policy"]
    gbs = pcfg["train_global_batch_size"]
    shuffle = bool((cfg.get("data") or {}).get("shuffle", True))
    loader = _ShardedPromptLoader(dataset, gbs, collate_fn, shuffle, a["seed"], rank, world)
    if resume and resume.get("dataloader"):
        loader.load_state_dict(torch.load(resume["dataloader"], weights_only=False))
    val_loader = None
    if val_dataset is not None and len(val_dataset):
        vb = max(world, (min(a["val_global_batch_size"], len(val_dataset)) // world) * world)
        val_loader = _ShardedPromptLoader(val_dataset, vb, collate_fn, False, 0, rank, world)
    if policy is None:
        if value_head and model_cfg is not None:
            model_cfg.value_head = True
        policy = PolicyWorker(pcfg, model_cfg=model_cfg, tokenizer=tokenizer, init_reference_model=needs_reference, seed=a["seed"])
        if resume and resume.get("weights"):
            policy.load_checkpoint(resume["weights"], resume.get("optimizer"))
    return policy, loader, val_loader, logger, checkpointer, save_state, cfg


def setup_sft(cfg, tokenizer, dataset, val_dataset, model_cfg=None, policy=None):
    """Returns (policy, loader, val_loader, loss_fn, logger, checkpointer, save_state, cfg)."""
    from functools import partial

    from rl_b200.data.collate import sft_collate_fn

    pad = tokenizer.pad_token_id if tokenizer is not None and tokenizer.pad_token_id is not None else 0
    s = dict(SFT_DEFAULTS)
    s.update(cfg.get("sft") or {})
    collate = partial(sft_collate_fn, pad_token_id=pad, only_unmask_final=s["only_unmask_final"],
                      make_sequence_length_divisible_by=cfg["policy"].get("make_sequence_length_divisible_by", 1))
    policy, loader, val_loader, logger, ck, ss, cfg = _setup_common(cfg, "sft", SFT_DEFAULTS, tokenizer, dataset, val_dataset, collate,
                                                                    model_cfg, False, False, policy)
    return policy, loader, val_loader, NLLLossFn(), logger, ck, ss, cfg


def setup_dpo(cfg, tokenizer, dataset, val_dataset, model_cfg=None, policy=None):
    from functools import partial

    from rl_b200.data.collate import preference_collate_fn

    pad = tokenizer.pad_token_id if tokenizer is not None and tokenizer.pad_token_id is not None else 0
    collate = partial(preference_collate_fn, pad_token_id=pad)
    policy, loader, val_loader, logger, ck, ss, cfg = _setup_common(cfg, "dpo", DPO_DEFAULTS, tokenizer, dataset, val_dataset, collate,
                                                                    model_cfg, True, False, policy)
    d = cfg["dpo"]
    loss = DPOLossFn({k: d[k] for k in ("reference_policy_kl_penalty", "preference_loss_weight", "sft_loss_weight",
                                        "preference_average_log_probs", "sft_average_log_probs")})
    return policy, loader, val_loader, loss, logger, ck, ss, cfg


def setup_rm(cfg, tokenizer, dataset, val_dataset, model_cfg=None, policy=None):
    from functools import partial

    from rl_b200.data.collate import preference_collate_fn

    pad = tokenizer.pad_token_id if tokenizer is not None and tokenizer.pad_token_id is not None else 0
    collate = partial(preference_collate_fn, pad_token_id=pad)
    policy, loader, val_loader, logger, ck, ss, cfg = _setup_common(cfg, "rm", RM_DEFAULTS, tokenizer, dataset, val_dataset, collate,
                                                                    model_cfg, False, True, policy)
    return policy, loader, val_loader, PreferenceLossFn(), logger, ck, ss, cfg


def add_ref_logprobs_to_data(policy, batch: BatchedDataDict, micro_batch_size: Optional[int] = None) -> BatchedDataDict:
    """DPO: log-probabilities of the frozen reference policy for every row (chosen and rejected)."""
    batch["reference_policy_logprobs"] = policy.get_reference_policy_logprobs(batch, micro_batch_size)["reference_logprobs"]
    return batch


def validate_supervised(policy, val_loader, loss_fn, cfg_alg: dict, step: int, logger: Optional[Logger], prefix: str = "validation",
                        preprocess: Optional[Callable] = None) -> dict:
    if val_loader is None:
        return {}
    sums: dict[str, float] = {}
    n = 0
    for i, batch in enumerate(val_loader):
        if i >= cfg_alg["val_batches"]:
            break
        if preprocess is not None:
            batch = preprocess(batch)
        mult = 2 if getattr(loss_fn, "requires_pairs", False) else 1
        res = policy.train(batch, loss_fn, eval_mode=True, gbs=batch.size * _world()[1], mbs=mult * cfg_alg["val_micro_batch_size"])
        m = _aggregate_train_metrics(res)
        for k, v in m.items():
            sums[k] = sums.get(k, 0.0) + v
        n += 1
    out = {k: v / max(1, n) for k, v in sums.items()}
    out = {("val_loss" if k == "loss" else k): v for k, v in out.items()}
    if logger is not None and out:
        logger.log_metrics(out, step, prefix=prefix)
    return out


def _supervised_train(policy, loader, val_loader, loss_fn, logger, checkpointer, save_state, cfg, key: str,
                      preprocess: Optional[Callable] = None, step_callback=None) -> dict:
    rank, world = _world()
    a, pcfg = cfg[key], cfg["policy"]
    timer = Timer()
    timeout = TimeoutChecker((cfg.get("checkpointing") or {}).get("checkpoint_must_save_by"), fit_last_save_time=True)
    total_steps, epoch = save_state["total_steps"], save_state["current_epoch"]
    last: dict = {}
    if a["val_at_start"] and total_steps == 0:
        validate_supervised(policy, val_loader, loss_fn, a, 0, logger, preprocess=preprocess)
    while epoch < a["max_num_epochs"] and total_steps < a["max_num_steps"]:
        for batch in loader:
            if total_steps >= a["max_num_steps"]:
                break
            with timer.time("total_step_time"):
                if preprocess is not None:
                    with timer.time("data_processing"):
                        batch = preprocess(batch)
                with timer.time("policy_training"):
                    policy.prepare_for_training()
                    mult = 2 if getattr(loss_fn, "requires_pairs", False) else 1  # preference rows come in pairs
                    res = policy.train(batch, loss_fn, gbs=mult * pcfg["train_global_batch_size"], mbs=mult * pcfg["train_micro_batch_size"])
            total_steps += 1
            metrics = _aggregate_train_metrics(res)
            tok = _all_reduce_scalars({"tokens": float(batch["input_lengths"].sum()), "n": float(batch.size)})
            metrics["total_num_tokens"] = tok["tokens"]
            is_last = total_steps >= a["max_num_steps"]
            val = {}
            if val_loader is not None and a["val_period"] > 0 and (total_steps % a["val_period"] == 0 or (is_last and a["val_at_end"])):
                val = validate_supervised(policy, val_loader, loss_fn, a, total_steps, logger, preprocess=preprocess)
                save_state["val_loss"] = val.get("val_loss")
            save_state.update(current_step=total_steps, total_steps=total_steps, current_epoch=epoch,
                              consumed_samples=save_state["consumed_samples"] + int(tok["n"]))
            timing = timer.get_timing_metrics("sum")
            timeout.mark_iteration()
            must = _agree_any(timeout.check_save())   # collective decision: saving is collective
            ck = cfg.get("checkpointing") or {}
            if checkpointer.enabled and (is_last or must or (ck.get("save_period") and total_steps % ck["save_period"] == 0)):
                save_checkpoint(policy, loader, checkpointer, save_state, cfg, total_steps, val)
            if logger is not None:
                logger.log_metrics(metrics, total_steps, prefix="train")
                logger.log_metrics(timing, total_steps, prefix="timing/train")
            if _is_main():
                extra = f" acc={metrics['accuracy']:.3f}" if "accuracy" in metrics else ""
                print(f"[{key}] step {total_steps}: loss={metrics['loss']:.5f}{extra} grad_norm={metrics['grad_norm']:.3f} "
                      f"tokens={int(tok['tokens'])} step_time={timing.get('total_step_time', 0):.2f}s", flush=True)
            last = {"train": metrics, "timing": timing, "validation": val}
            if step_callback is not None:
                step_callback(total_steps, last)
            _ft_beat(total_steps)
            timer.reset()
            if must:
                return last
        epoch += 1
        save_state["current_epoch"] = epoch
    return last


def sft_train(policy, loader, val_loader, tokenizer, loss_fn, logger, checkpointer, save_state, cfg, step_callback=None) -> dict:
    return _supervised_train(policy, loader, val_loader, loss_fn, logger, checkpointer, save_state, cfg, "sft", None, step_callback)


def dpo_train(policy, loader, val_loader, tokenizer, loss_fn, logger, checkpointer, save_state, cfg, step_callback=None) -> dict:
    mbs = cfg["policy"].get("logprob_batch_size")
    return _supervised_train(policy, loader, val_loader, loss_fn, logger, checkpointer, save_state, cfg, "dpo",
                             lambda b: add_ref_logprobs_to_data(policy, b, mbs), step_callback)


def rm_train(policy, loader, val_loader, tokenizer, loss_fn, logger, checkpointer, save_state, cfg, step_callback=None) -> dict:
    return _supervised_train(policy, loader, val_loader, loss_fn, logger, checkpointer, save_state, cfg, "rm", None, step_callback)
