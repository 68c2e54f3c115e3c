"""GRPO / DAPO / GSPO training loop (``setup`` + ``grpo_train`` + ``validate``).

Phases and timer names follow nemo_rl/algorithms/grpo.py:2682-3819: data_processing -> prepare_for_generation (refit)
-> generation (multi-turn rollouts + rewards) -> reward shaping / scaling / dynamic sampling -> policy and reference
log-probabilities -> advantages -> policy_training -> validation / checkpoint / metrics.

Runtime model: SPMD. Every rank (one per GPU) executes this loop on its own slice of the prompts with its own
colocated generation engine; all responses to one prompt live on one rank, so group baselines are local, and the
only cross-rank traffic is the optimizer's gradient exchange plus a few scalar all-reduces for metrics. With the
trainer and the engine sharing one set of weight buffers the refit step is a pointer hand-off.
"""

from __future__ import annotations

import math
import os
import time
from typing import Any, Callable, Optional

import numpy as np
import torch

from rl_b200.distributed.ft_launcher import beat as _ft_beat
import torch.distributed as dist

from rl_b200.algorithms.advantage_estimator import create_advantage_estimator
from rl_b200.algorithms.loss.loss_functions import ClippedPGLossFn
from rl_b200.algorithms.reward_functions import apply_reward_shaping, scale_rewards
from rl_b200.algorithms.utils import calculate_baseline_and_std_per_prompt, compute_performance_metrics, set_seed
from rl_b200.data.llm_message_utils import batched_message_log_to_flat_message, multimodal_fields
from rl_b200.distributed.batched_data_dict import BatchedDataDict
from rl_b200.experience.rollouts import run_multi_turn_rollout
from rl_b200.utils.checkpoint import CheckpointManager
from rl_b200.utils.logger import Logger
from rl_b200.utils.profiling import maybe_gpu_profile_step
from rl_b200.utils.timer import TimeoutChecker, Timer

GRPO_DEFAULTS = dict(
    num_prompts_per_step=32,
    num_generations_per_prompt=16,
    max_num_epochs=1,
    max_num_steps=1_000_000,
    max_rollout_turns=1,
    normalize_rewards=True,
    use_leave_one_out_baseline=True,
    advantage_clip_low=None,
    advantage_clip_high=None,
    val_period=10,
    val_start_at=-1,
    val_batch_size=256,
    val_at_start=False,
    val_at_end=False,
    max_val_samples=256,
    val_num_generations_per_prompt=1,
    stop_at_validation_metric=None,
    stop_at_validation_threshold=None,
    skip_reference_policy_logprobs_calculation=False,
    seed=42,
    overlong_filtering=False,
    use_dynamic_sampling=False,
    dynamic_sampling_max_gen_batches=10,
    batch_multiplier=1.0,
    reward_shaping=None,
    reward_scaling=None,
    calculate_advantages_on_gpu=False,
    seq_logprob_error_threshold=None,
    adv_estimator=None,
    async_grpo=None,
)


def _world():
    """(data-parallel rank, data-parallel size): the coordinates that shard data. Ranks of one model-parallel group
    (tensor / pipeline / context) share a data-parallel rank and therefore see the same samples."""
    from rl_b200.parallel.state import get_state

    st = get_state()
    if st.world > 1:
        return st.dp_rank, st.dp
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


def _dp_group():
    from rl_b200.parallel.state import get_state

    st = get_state()
    if st.world > 1 and st.tp * st.pp * st.cp > 1:
        return st.dp_group if st.dp > 1 else "self"
    return None


def _agree_any(flag: bool) -> bool:
    """True on every rank of the job if ``flag`` is true on any rank (world group, MAX)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return bool(flag)
    t = torch.tensor([1 if flag else 0], dtype=torch.int32)
    if torch.cuda.is_available() and dist.get_backend() == "nccl":
        t = t.cuda()
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return bool(t.item())


def _is_main() -> bool:
    return not (dist.is_available() and dist.is_initialized()) or dist.get_rank() == 0


def _all_reduce_scalars(values: dict[str, float], op: str = "sum") -> dict[str, float]:
    """Combines per-rank scalars over the data-parallel ranks."""
    rank, world = _world()
    group = _dp_group()
    if world == 1 or group == "self":
        return dict(values)
    keys = sorted(values)
    t = torch.tensor([float(values[k]) for k in keys], dtype=torch.float64)
    if torch.cuda.is_available() and dist.get_backend() == "nccl":
        t = t.cuda()
    dist.all_reduce(t, op={"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN}[op], group=group)
    return {k: float(v) for k, v in zip(keys, t.tolist())}


class _ShardedPromptLoader:
    """Iterates a dataset in global batches of ``global_batch`` prompts and hands each rank its contiguous slice.
    Shuffling uses a seeded permutation per epoch so that every rank sees the same order; the position is
    checkpointable (``state_dict`` / ``load_state_dict``)."""

    def __init__(self, dataset, global_batch: int, collate_fn: Callable, shuffle: bool, seed: int, rank: int, world: int,
                 drop_last: bool = True):
        assert global_batch % world == 0, f"{global_batch} prompts per step do not split over {world} ranks"
        self.ds, self.gb, self.collate, self.shuffle, self.seed = dataset, global_batch, collate_fn, shuffle, seed
        self.rank, self.world = rank, world
        self.epoch, self.pos = 0, 0

    def __len__(self):
        return len(self.ds) // self.gb

    def _order(self):
        n = len(self.ds)
        if not self.shuffle:
            return list(range(n))
        g = torch.Generator().manual_seed(self.seed + self.epoch)
        return torch.randperm(n, generator=g).tolist()

    def __iter__(self):
        order = self._order()
        per = self.gb // self.world
        while self.pos + self.gb <= len(order):
            idx = order[self.pos + self.rank * per : self.pos + (self.rank + 1) * per]
            self.pos += self.gb
            yield self.collate([self.ds[i] for i in idx])
        self.pos = 0
        self.epoch += 1

    def state_dict(self):
        return {"epoch": self.epoch, "pos": self.pos}

    def load_state_dict(self, sd):
        self.epoch, self.pos = int(sd["epoch"]), int(sd["pos"])


def default_save_state() -> dict:
    return {"current_step": 0, "current_epoch": 0, "total_steps": 0, "consumed_samples": 0, "total_valid_tokens": 0, "val_reward": -99999999.0}


def setup(master_config: dict, tokenizer, dataset, val_dataset, task_to_env: dict, val_task_to_env: Optional[dict] = None,
          model_cfg=None, policy=None, build_generation: bool = True):
    """Builds everything ``grpo_train`` needs: policy worker (+ colocated engine), loaders, loss, logger, checkpointer.

    Returns ``(policy, generation, dataloader, val_dataloader, loss_fn, logger, checkpointer, save_state, master_config)``.
    """
    from rl_b200.data.collate import rl_collate_fn
    from rl_b200.policy.worker import PolicyWorker

    from rl_b200.policy.worker import ensure_parallel

    ensure_parallel(master_config["policy"])
    rank, world = _world()
    cfg = master_config
    g = dict(GRPO_DEFAULTS)
    g.update(cfg.get("grpo") or {})
    cfg["grpo"] = g
    set_seed(g["seed"] + rank)
    logger = Logger(cfg.get("logger"), is_main=_is_main())
    if _is_main():
        logger.log_hyperparams(cfg)
    checkpointer = CheckpointManager(cfg.get("checkpointing"))
    save_state = default_save_state()
    resume = checkpointer.get_resume_paths() if checkpointer.enabled else None
    if resume:
        info = checkpointer.load_training_info(resume["root"])
        if info:
            save_state.update(info)
    loader = _ShardedPromptLoader(dataset, g["num_prompts_per_step"], rl_collate_fn, bool((cfg.get("data") or {}).get("shuffle", True)),
                                  g["seed"], rank, world)
    if resume and resume.get("dataloader"):
        loader.load_state_dict(torch.load(resume["dataloader"], weights_only=False))
    val_loader = None
    if val_dataset is not None and len(val_dataset):
        vb = max(world, (min(g["val_batch_size"], len(val_dataset)) // world) * world)
        val_loader = _ShardedPromptLoader(val_dataset, vb, rl_collate_fn, False, 0, rank, world)
    pcfg = cfg["policy"]
    if policy is None:
        needs_ref = (cfg.get("loss_fn") or {}).get("reference_policy_kl_penalty", 0.01) != 0 and not g["skip_reference_policy_logprobs_calculation"]
        policy = PolicyWorker(pcfg, model_cfg=model_cfg, tokenizer=tokenizer, init_reference_model=needs_ref, seed=g["seed"],
                              weights_path=None)
        if resume and resume.get("weights"):
            policy.load_checkpoint(resume["weights"], resume.get("optimizer"))
    # training ranks of a split job have no engine: generation runs on other ranks (rl_b200/algorithms/noncolocated.py)
    generation = policy.build_generation(pcfg.get("generation")) if build_generation else None
    loss_fn = ClippedPGLossFn(cfg.get("loss_fn"))
    return policy, generation, loader, val_loader, loss_fn, logger, checkpointer, save_state, cfg


# ---------------------------------------------------------------------------------------------- helpers
def refit_policy_generation(policy, generation, timer: Optional[Timer] = None) -> None:
    """Makes the engine serve the trainer's current weights. Colocated at matching layout both sides address the same
    buffers, so only the engine's request state is reset; other layouts go through :mod:`rl_b200.refit`."""
    sync = getattr(policy, "weight_synchronizer", None)
    if sync is not None:
        eng = getattr(generation, "engine", None)
        if getattr(eng, "quantization", None) == "fp8" and getattr(eng, "tpw", 1) == 1 and hasattr(sync, "sync_weights_fp8"):
            # block-128 FP8 rollout: the re-shard pass quantises on the way (one read of the trainer's weights, fp8 bytes
            # over NVLink) and the engine takes the quantised copies as they are
            sync.sync_weights_fp8()
            eng.quantized_by_refit = True
        else:
            sync.sync_weights(timer)
    generation.prepare_for_generation()


def build_train_data(batch: BatchedDataDict, pad_token_id: int, make_divisible_by: int = 1) -> BatchedDataDict:
    """Flattens message logs into the ClippedPG train batch: ``input_ids``, ``input_lengths``, ``token_mask`` (1 on
    generated tokens), ``sample_mask`` (loss multiplier), ``generation_logprobs``."""
    for log in batch["message_log"]:
        for m in log:
            n = m["token_ids"].numel()
            if m["role"] == "assistant":
                m["token_loss_mask"] = torch.ones(n, dtype=torch.long)
                if "generation_logprobs" not in m:
                    m["generation_logprobs"] = torch.zeros(n, dtype=torch.float32)
            else:
                m["token_loss_mask"] = torch.zeros(n, dtype=torch.long)
                m["generation_logprobs"] = torch.zeros(n, dtype=torch.float32)
    flat, lengths = batched_message_log_to_flat_message(batch["message_log"], {"token_ids": pad_token_id}, make_divisible_by)
    extra = {}
    traces = batch.get("routed_experts")
    if traces is not None and len(traces) and all(t is not None for t in traces):
        # the engine's routing decisions per position (rollout routing replay): aligned with input_ids, -1 where unknown
        S = flat["token_ids"].shape[1]
        re = torch.full((len(traces), S) + tuple(traces[0].shape[1:]), -1, dtype=torch.int16)
        for i, t in enumerate(traces):
            re[i, : min(S, t.shape[0])] = t[:S]
        extra["routed_experts"] = re
    return BatchedDataDict(
        input_ids=flat["token_ids"], input_lengths=lengths, token_mask=flat["token_loss_mask"].float(),
        sample_mask=batch["loss_multiplier"].float().clone(), generation_logprobs=flat["generation_logprobs"].float(),
        **multimodal_fields(flat), **extra,
    )


def dynamic_sampling(repeated: BatchedDataDict, std: torch.Tensor, baseline: torch.Tensor, cache: Optional[BatchedDataDict],
                     num_prompts_local: int, n_gen: int):
    """DAPO: keep only prompts whose responses disagree (std > 0), accumulate across generation rounds until enough
    prompts are collected. Returns (batch or None when more rounds are needed, cache, stats)."""
    keep = (std > 0).nonzero(as_tuple=True)[0].tolist()
    kept = repeated.select_indices(keep)
    kept["_baseline"] = baseline[keep]
    kept["_std"] = std[keep]
    cache = kept if cache is None or cache.size == 0 else BatchedDataDict.from_batches([cache, kept])
    need = num_prompts_local * n_gen
    stats = {"dynamic_sampling_kept_fraction": len(keep) / max(1, len(std)), "dynamic_sampling_cached": cache.size}
    if cache.size >= need:
        return cache.slice(0, need), None, stats
    return None, cache, stats


def compute_and_apply_seq_logprob_error_masking(train_data: BatchedDataDict, threshold: Optional[float]) -> dict:
    """Masks sequences whose mean |trainer - generator| log-prob gap exceeds the threshold (engine / trainer drift)."""
    if threshold is None:
        return {}
    tm = train_data["token_mask"][:, 1:]
    err = ((train_data["prev_logprobs"][:, 1:] - train_data["generation_logprobs"][:, 1:]).abs() * tm).sum(-1) / tm.sum(-1).clamp(min=1)
    bad = err > threshold
    train_data["sample_mask"] = train_data["sample_mask"] * (~bad).float()
    return {"seq_logprob_error_masked_fraction": float(bad.float().mean()), "seq_logprob_error_max": float(err.max()) if err.numel() else 0.0}


def _aggregate_train_metrics(res: dict) -> dict[str, float]:
    """Micro-batch metrics are pre-normalised by global counts: sums over micro-batches and ranks are global means;
    min / max style keys reduce with min / max."""
    mm = res["all_mb_metrics"]
    sums, mins, maxs = {}, {}, {}
    for k, v in mm.items():
        if k in ("lr", "global_valid_seqs", "global_valid_toks"):
            sums[k] = float(np.mean(v))
        elif k.endswith("_min"):
            mins[k] = float(np.min(v))
        elif k.endswith("_max"):
            maxs[k] = float(np.max(v))
        else:
            sums[k] = float(np.sum(v))
    rank, world = _world()
    keep_local = {k: sums.pop(k) for k in ("lr", "global_valid_seqs", "global_valid_toks") if k in sums}
    out = _all_reduce_scalars(sums, "sum")
    out.update(_all_reduce_scalars(mins, "min"))
    out.update(_all_reduce_scalars(maxs, "max"))
    out.update(keep_local)
    n_steps = max(1, len(res["loss"]))
    # sums ran over every optimizer step of the call; report the per-step mean
    for k in list(out):
        if k not in keep_local and not k.endswith(("_min", "_max")) and k != "num_valid_samples":
            out[k] = out[k] / n_steps
    out["loss"] = float(res["loss"].mean()) if len(res["loss"]) else 0.0
    out["grad_norm"] = float(res["grad_norm"].mean()) if len(res["grad_norm"]) else 0.0
    return out


# ---------------------------------------------------------------------------------------------- validation
def validate(policy, generation, val_loader, tokenizer, task_to_env, step: int, master_config: dict, logger: Optional[Logger] = None):
    if val_loader is None:
        return {}, {}
    g = master_config["grpo"]
    timer = Timer()
    rewards, lengths = [], []
    pad = tokenizer.pad_token_id if tokenizer is not None and tokenizer.pad_token_id is not None else 0
    with timer.time("total_validation_time"):
        refit_policy_generation(policy, generation)
        seen = 0
        for batch in val_loader:
            n_gen = g["val_num_generations_per_prompt"]
            if n_gen > 1:
                batch = batch.repeat_interleave(n_gen)
                batch["message_log"] = [[dict(m) for m in log] for log in batch["message_log"]]
            batch, m = run_multi_turn_rollout(generation, batch, tokenizer, task_to_env, master_config["policy"]["max_total_sequence_length"],
                                              g["max_rollout_turns"], greedy=False, pad_token_id=pad)
            rewards.append(batch["total_reward"])
            lengths.append(batch["generation_lengths"].float())
            seen += batch.size * _world()[1]
            if seen >= g["max_val_samples"]:
                break
        generation.finish_generation()
    r = torch.cat(rewards) if rewards else torch.zeros(0)
    L = torch.cat(lengths) if lengths else torch.zeros(0)
    agg = _all_reduce_scalars({"r_sum": float(r.sum()), "n": float(r.numel()), "l_sum": float(L.sum())})
    val = {"accuracy": agg["r_sum"] / max(1.0, agg["n"]), "avg_length": agg["l_sum"] / max(1.0, agg["n"])}
    timing = timer.get_timing_metrics("sum")
    if logger is not None:
        logger.log_metrics(val, step, prefix="validation")
        logger.log_metrics(timing, step, prefix="timing/validation")
    return val, timing


# ---------------------------------------------------------------------------------------------- the loop
def grpo_train(policy, generation, dataloader, val_dataloader, tokenizer, loss_fn, task_to_env, val_task_to_env, logger,
               checkpointer, save_state: dict, master_config: dict, step_callback: Optional[Callable[[int, dict], None]] = None,
               teacher_groups=None) -> dict:
    """Runs GRPO until ``max_num_steps`` / ``max_num_epochs``. Returns the last step's metrics. ``teacher_groups``:
    ``(alias -> TeacherGroup, alias -> serving alias)`` for on-policy distillation (built from the config when absent)."""
    rank, world = _world()
    cfg = master_config
    g, pcfg = cfg["grpo"], cfg["policy"]
    loss_cfg = cfg.get("loss_fn") or {}
    timer = Timer()
    timeout = TimeoutChecker((cfg.get("checkpointing") or {}).get("checkpoint_must_save_by"), fit_last_save_time=True)
    adv_estimator = create_advantage_estimator(g, loss_cfg)
    pad = tokenizer.pad_token_id if tokenizer is not None and tokenizer.pad_token_id is not None else 0
    n_gen = g["num_generations_per_prompt"]
    n_prompts_local = g["num_prompts_per_step"] // world
    use_ref = loss_fn.cfg["reference_policy_kl_penalty"] != 0 and not g["skip_reference_policy_logprobs_calculation"]
    step = save_state["current_step"]
    total_steps = save_state["total_steps"]
    val_task_to_env = val_task_to_env or task_to_env
    last_metrics: dict = {}
    # rollouts owned by a gym (env.should_use_nemo_gym): rows go to the agent server named by env.nemo_gym.url, which calls the
    # policy server at env.nemo_gym.policy_base_url (engine/http_server.py)
    gym_client = None
    env_cfg = cfg.get("env") or {}
    if env_cfg.get("should_use_nemo_gym"):
        from rl_b200.experience.gym_rollouts import GymClient

        gcfg = env_cfg.get("nemo_gym") or {}
        gym_client = task_to_env.get("nemo_gym_client") if isinstance(task_to_env, dict) and "nemo_gym_client" in task_to_env else GymClient(
            gcfg["url"], gcfg["policy_base_url"], float(gcfg.get("timeout_s", 1800.0)), int(gcfg.get("max_retries", 2)))
    # on-policy distillation (grpo.adv_estimator.name: opd): frozen teachers, one per distinct checkpoint
    opd_groups = teacher_groups
    opd_metrics: dict = {}
    if opd_groups is None and (g.get("adv_estimator") or {}).get("name") == "opd":
        from rl_b200.algorithms import opd as _opd

        opd_groups = _opd.create_teacher_groups(cfg, tokenizer, getattr(policy, "model_cfg", None))

    if g["val_at_start"] and step == 0:
        validate(policy, generation, val_dataloader, tokenizer, val_task_to_env, 0, cfg, logger)

    epoch = save_state["current_epoch"]
    while epoch < g["max_num_epochs"] and total_steps < g["max_num_steps"]:
        ds_cache = None
        ds_rounds = 0
        for batch in dataloader:
            if total_steps >= g["max_num_steps"]:
                break
            maybe_gpu_profile_step(total_steps + 1, dist.get_rank() if dist.is_initialized() else 0)
            with timer.time("total_step_time"):
                # ---- data
                with timer.time("data_processing"):
                    repeated = batch.repeat_interleave(n_gen)
                    repeated["message_log"] = [[dict(m) for m in log] for log in repeated["message_log"]]
                    # random streams keyed by (global sample index, turn): rollouts do not depend on the rank layout
                    repeated["rng_ids"] = repeated["idx"] * n_gen + torch.arange(n_gen).repeat(batch.size)
                    prompt_flat, prompt_lens = batched_message_log_to_flat_message(repeated["message_log"], {"token_ids": pad})
                    prompt_ids = prompt_flat["token_ids"]
                # ---- refit + generation
                with timer.time("prepare_for_generation/total"):
                    refit_policy_generation(policy, generation, timer)
                with timer.time("generation"):
                    if gym_client is not None:
                        # the gym owns the episodes (turns, tools, verification) and calls the policy's HTTP endpoint
                        from rl_b200.experience.gym_rollouts import run_gym_rollout_sync

                        repeated, rollout_metrics = run_gym_rollout_sync(
                            repeated, gym_client, tokenizer, n_gen, max_seq_len=pcfg["max_total_sequence_length"],
                            reward_penalty_config=cfg.get("reward_penalties"), sampling=dict(temperature=(pcfg.get("generation") or {}).get("temperature", 1.0)))
                        rollout_metrics = {k: v for k, v in rollout_metrics.items() if isinstance(v, (int, float))}
                        repeated["generation_lengths"] = torch.tensor([sum(int(m["token_ids"].numel()) for m in log if m["role"] == "assistant")
                                                                       for log in repeated["message_log"]])
                    else:
                        repeated, rollout_metrics = run_multi_turn_rollout(
                            generation, repeated, tokenizer, task_to_env, pcfg["max_total_sequence_length"], g["max_rollout_turns"],
                            greedy=False, pad_token_id=pad)
                    generation.finish_generation()
                # ---- rewards
                with timer.time("reward_calculation"):
                    repeated = scale_rewards(repeated, g.get("reward_scaling"))
                    repeated = apply_reward_shaping(repeated, g.get("reward_shaping"))
                    rewards = repeated["total_reward"].float()
                    repeated["_prompt_ids"] = prompt_ids
                    valid = torch.ones_like(rewards)
                    baseline, std = calculate_baseline_and_std_per_prompt(prompt_ids, rewards, valid, g["use_leave_one_out_baseline"])
                    if g["use_dynamic_sampling"]:
                        ds_rounds += 1
                        ready, ds_cache, ds_stats = dynamic_sampling(repeated, std, baseline, ds_cache, n_prompts_local, n_gen)
                        rollout_metrics.update(ds_stats)
                        enough = _all_reduce_scalars({"ready": 1.0 if ready is not None else 0.0}, "min")["ready"] > 0
                        if not enough:
                            if ds_rounds >= g["dynamic_sampling_max_gen_batches"]:
                                raise RuntimeError("dynamic sampling: not enough prompts with non-zero reward std after "
                                                   f"{ds_rounds} generation rounds")
                            continue
                        if ready is None:  # this rank is short while others are ready: pad by re-using what it has
                            ready = ds_cache.slice(0, min(ds_cache.size, n_prompts_local * n_gen))
                        repeated, ds_cache, ds_rounds = ready, None, 0
                        rewards = repeated["total_reward"].float()
                        prompt_ids = repeated["_prompt_ids"]
                    if g["overlong_filtering"]:
                        repeated["loss_multiplier"] = repeated["loss_multiplier"] * (~repeated["truncated"].bool()).float()
                # ---- train batch
                with timer.time("data_processing"):
                    train_data = build_train_data(repeated, pad, pcfg.get("make_sequence_length_divisible_by", 1))
                    train_data["rewards"] = rewards
                # ---- log-probabilities under the pre-update and the reference policy
                with timer.time("policy_and_reference_logprobs"):
                    policy.prepare_for_lp_inference()
                    if loss_fn.cfg["force_on_policy_ratio"]:
                        train_data["prev_logprobs"] = train_data["generation_logprobs"].clone()
                    else:
                        train_data["prev_logprobs"] = policy.get_logprobs(train_data)["logprobs"]
                    if use_ref:
                        train_data["reference_policy_logprobs"] = policy.get_reference_policy_logprobs(train_data)["reference_logprobs"]
                    else:
                        train_data["reference_policy_logprobs"] = torch.zeros_like(train_data["prev_logprobs"])
                    mask_metrics = compute_and_apply_seq_logprob_error_masking(train_data, g["seq_logprob_error_threshold"])
                # ---- advantages
                with timer.time("advantage_calculation"):
                    tm = train_data["token_mask"]
                    extra = {}
                    if opd_groups is not None:   # on-policy distillation: every sample is scored by its agent's teacher
                        from rl_b200.algorithms import opd as _opd

                        with timer.time("teacher_logprob_inference"):
                            agents = repeated.get("agent_ref") or repeated.get("task_name") or [None] * train_data.size
                            extra["teacher_logprobs"], opd_metrics = _opd.compute_teacher_logprobs(
                                train_data, agents, opd_groups[0], opd_groups[1], _opd.opd_cfg(cfg))
                    adv = adv_estimator.compute_advantage(
                        prompt_ids, rewards, tm, valid_mask=torch.ones_like(rewards),
                        reward_components=repeated.get("reward_components"), logprobs_policy=train_data["prev_logprobs"],
                        logprobs_reference=train_data["reference_policy_logprobs"], dp_group=_dp_group(), **extra)
                    if isinstance(adv, tuple):
                        adv = adv[0]
                    lo, hi = g["advantage_clip_low"], g["advantage_clip_high"]
                    if lo is not None or hi is not None:
                        adv = adv.clamp(min=lo, max=hi)
                    train_data["advantages"] = adv
                # ---- training
                with timer.time("policy_training"):
                    policy.prepare_for_training()
                    res = policy.train(train_data, loss_fn, gbs=pcfg["train_global_batch_size"], mbs=pcfg["train_micro_batch_size"])
                    policy.finish_training()
                step += 1
                total_steps += 1
            # ---- validation / checkpoint / metrics (outside the step timer, as in the reference's accounting)
            is_last = total_steps >= g["max_num_steps"]
            val_metrics = {}
            if val_dataloader is not None and g["val_period"] > 0 and (total_steps % g["val_period"] == 0 or (is_last and g["val_at_end"])):
                val_metrics, _ = validate(policy, generation, val_dataloader, tokenizer, val_task_to_env, total_steps, cfg, logger)
                save_state["val_reward"] = val_metrics.get("accuracy", save_state["val_reward"])
            tm1 = train_data["token_mask"][:, 1:] * train_data["sample_mask"][:, None]
            counts = _all_reduce_scalars({
                "reward_sum": float(rewards.sum()), "n": float(rewards.numel()), "valid_tokens": float(tm1.sum()),
                "total_tokens": float(train_data["input_lengths"].sum()), "generated_tokens": float(repeated["generation_lengths"].sum()),
                "adv_abs_sum": float((train_data["advantages"][:, 1:].abs() * tm1).sum()),
            })
            metrics = _aggregate_train_metrics(res)
            metrics.update({
                "reward": counts["reward_sum"] / max(1.0, counts["n"]),
                "mean_prompt_length": float(prompt_lens.float().mean()),
                "total_num_tokens": counts["total_tokens"],
                "mean_abs_advantage": counts["adv_abs_sum"] / max(1.0, counts["valid_tokens"]),
                **{k: v for k, v in rollout_metrics.items() if isinstance(v, (int, float))},
                **mask_metrics,
                **opd_metrics, **(getattr(adv_estimator, "last_metrics", None) or {}),
            })
            save_state.update(current_step=step, total_steps=total_steps, current_epoch=epoch,
                              consumed_samples=save_state["consumed_samples"] + int(counts["n"]),
                              total_valid_tokens=save_state["total_valid_tokens"] + int(counts["valid_tokens"]))
            timing = timer.get_timing_metrics("sum")
            perf = compute_performance_metrics(timing, num_gpus=world, total_tokens=int(counts["total_tokens"]),
                                               generated_tokens=int(counts["generated_tokens"]))
            timeout.mark_iteration()
            ck = cfg.get("checkpointing") or {}
            # every rank must take the same branch: saving is collective, and each rank's wall clock differs
            must = _agree_any(timeout.check_save())
            if checkpointer.enabled and (is_last or must or (ck.get("save_period") and total_steps % ck["save_period"] == 0)):
                with timer.time("checkpointing"):
                    save_checkpoint(policy, dataloader, checkpointer, save_state, cfg, total_steps, val_metrics)
            if logger is not None:
                logger.log_metrics(metrics, total_steps, prefix="train")
                logger.log_metrics(timing, total_steps, prefix="timing/train")
                logger.log_metrics(perf, total_steps, prefix="performance")
            if _is_main():
                print(f"[grpo] step {total_steps}: loss={metrics['loss']:.5f} reward={metrics['reward']:.4f} "
                      f"mult_prob_err={metrics.get('token_mult_prob_error', float('nan')):.4f} "
                      f"step_time={timing.get('total_step_time', 0):.2f}s gen={timing.get('generation', 0):.2f}s "
                      f"lp={timing.get('policy_and_reference_logprobs', 0):.2f}s train={timing.get('policy_training', 0):.2f}s "
                      f"tok/s/gpu={perf.get('tokens_per_sec_per_gpu', 0):.0f}", flush=True)
            last_metrics = {"train": metrics, "timing": timing, "performance": perf, "validation": val_metrics}
            if step_callback is not None:
                step_callback(total_steps, last_metrics)
            _ft_beat(total_steps)
            timer.reset()
            thr = g.get("stop_at_validation_threshold")
            if thr is not None and val_metrics and val_metrics.get("accuracy", -1e9) >= thr:
                return last_metrics
            if must:
                return last_metrics
        epoch += 1
        save_state["current_epoch"] = epoch
    return last_metrics


def save_checkpoint(policy, dataloader, checkpointer: CheckpointManager, save_state: dict, cfg: dict, step: int,
                    val_metrics: Optional[dict] = None, extra_files: Optional[dict] = None) -> None:
    """``extra_files``: name -> picklable object written beside the dataloader state by every data-parallel rank that owns
    one (``replay_buffer.pt`` of the off-policy trainers; rank r > 0 writes ``name.rank{r}``)."""
    rank, world = _world()
    ck = cfg.get("checkpointing") or {}
    info = dict(save_state)
    if val_metrics:
        info["val"] = val_metrics
    tmp = None
    if _is_main():
        tmp = str(checkpointer.init_tmp_checkpoint(step, info, cfg))
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        box = [tmp]
        dist.broadcast_object_list(box, src=0)
        tmp = box[0]
    policy.save_checkpoint(
        os.path.join(tmp, "policy", "weights"),
        os.path.join(tmp, "policy", "optimizer") if ck.get("save_optimizer", True) else None,
        os.path.join(tmp, "policy", "tokenizer"),
        model_save_format=ck.get("model_save_format", "safetensors"))
    for name, obj in (extra_files or {}).items():
        torch.save(obj, os.path.join(tmp, name if rank == 0 else f"{name}.rank{rank}"))
    # all ranks of the job (tensor / pipeline / expert ranks included) have written their shards before the rename
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()
    if _is_main():
        torch.save(dataloader.state_dict(), os.path.join(tmp, "train_dataloader.pt"))
        checkpointer.finalize_checkpoint(tmp)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()
