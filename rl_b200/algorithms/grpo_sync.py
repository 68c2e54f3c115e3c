"""Synchronous GRPO with every sample travelling through the data plane.

The loop of :func:`rl_b200.algorithms.grpo.grpo_train`, but the driver never holds the training tensors: the rollout actor
stores each trajectory as one record under a step partition, the driver reads only the small fields it needs (rewards,
prompt ids, lengths, masks) to compute advantages and the seq-logprob-error statistics, writes the derived fields back, and
hands the policy a :class:`BatchMeta` (keys + lengths), from which every data-parallel rank fetches exactly its own shard.
The partition is cleared when the step ends. This is the structure of the reference's TransferQueue-mediated trainer
(nemo_rl/algorithms/grpo_sync.py:380-1400), its ``TQPolicy`` facade (nemo_rl/models/policy/tq_policy.py:84-603) and its
``SyncRolloutActor`` (nemo_rl/experience/sync_rollout_actor.py:108-425); the data plane here is
:mod:`rl_b200.data_plane` (in-process or TCP-store adapter) instead of TransferQueue.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Iterable, Optional, Sequence

import torch

from rl_b200.algorithms.advantage_estimator import create_advantage_estimator
from rl_b200.algorithms.async_grpo import _collect
from rl_b200.algorithms.grpo import _aggregate_train_metrics, _is_main, _world, build_train_data, refit_policy_generation
from rl_b200.data_plane import LocalDataPlane, SampleMeta, preshard
from rl_b200.data_plane.codec import batch_to_records, records_to_batch
from rl_b200.data_plane.interfaces import DataPlaneClient
from rl_b200.data_plane.worker_mixin import fetch_batch
from rl_b200.distributed.batched_data_dict import BatchedDataDict
from rl_b200.utils.timer import Timer

# fields of a stored trajectory
ROLLOUT_FIELDS = ("input_ids", "input_lengths", "token_mask", "sample_mask", "generation_logprobs", "total_reward", "prompt_ids",
                  "prompt_idx", "truncated")
JAGGED = ("input_ids", "token_mask", "generation_logprobs", "prev_logprobs", "reference_policy_logprobs", "advantages", "prompt_ids")
TRAIN_FIELDS = ("input_ids", "input_lengths", "token_mask", "sample_mask", "generation_logprobs", "prev_logprobs",
                "reference_policy_logprobs", "advantages")
DRIVER_FIELDS = ("input_lengths", "token_mask", "sample_mask", "total_reward", "prompt_ids", "prompt_idx", "truncated")


@dataclass
class BatchMeta:
    """What travels between driver and policy instead of tensors: the keys of a partition's samples, their token counts
    (for balanced sharding) and the fields known to be present (KVBatchMeta of the reference's data plane)."""

    partition: str
    keys: list[str]
    num_tokens: list[int]
    groups: list[str]
    fields: set = field(default_factory=set)

    @property
    def size(self) -> int:
        return len(self.keys)

    def select(self, idx: Sequence[int]) -> "BatchMeta":
        return BatchMeta(self.partition, [self.keys[i] for i in idx], [self.num_tokens[i] for i in idx], [self.groups[i] for i in idx],
                         set(self.fields))

    def sample_metas(self) -> list[SampleMeta]:
        return [SampleMeta(k, num_tokens=n, group=g) for k, n, g in zip(self.keys, self.num_tokens, self.groups)]


class SyncRolloutActor:
    """Runs the rollouts of one prompt batch and stores the trajectories in the data plane, one record per sample
    (``rollout_to_tq`` of the reference's actor). Returns the partition's :class:`BatchMeta` and the rollout metrics."""

    def __init__(self, policy, generation, tokenizer, task_to_env, cfg: dict, plane: DataPlaneClient, timer: Optional[Timer] = None):
        self.policy, self.generation, self.tokenizer, self.envs, self.cfg, self.plane = policy, generation, tokenizer, task_to_env, cfg, plane
        self.pad = tokenizer.pad_token_id if tokenizer is not None and tokenizer.pad_token_id is not None else 0
        self.timer = timer or Timer()
        self.rank, self.world = _world()

    def rollout_to_plane(self, batch: BatchedDataDict, partition: str, weight_version: int = 0) -> tuple[BatchMeta, dict]:
        traj, metrics = _collect(self.policy, self.generation, batch, self.tokenizer, self.envs, self.cfg, self.pad, self.timer)
        td = build_train_data(traj, self.pad)
        td["total_reward"] = traj["total_reward"].float()
        td["prompt_ids"] = traj["_prompt_ids"]
        td["prompt_idx"] = traj["idx"]
        td["truncated"] = traj["truncated"].float() if "truncated" in traj else torch.zeros(td.size)
        plen = (traj["_prompt_ids"] != self.pad).sum(-1) if traj["_prompt_ids"].dim() == 2 else None
        recs = batch_to_records(td, jagged=("input_ids", "token_mask", "generation_logprobs"))
        keys, ntok, groups = [], [], []
        for i, r in enumerate(recs):
            if plen is not None:   # prompt ids are stored without their padding, like every variable-length field
                r["prompt_ids"] = r["prompt_ids"][: int(plen[i])].clone()
            r["__jagged__"] = list(JAGGED)   # names of the variable-length fields a record may carry (now or later)
            key = f"{partition}/r{self.rank:03d}/{i:05d}"
            grp = f"{self.rank}:{int(r['prompt_idx'])}"
            self.plane.put(key, r, SampleMeta(key, num_tokens=int(r["input_lengths"]), weight_version=weight_version, group=grp,
                                              extra={"partition": partition}))
            keys.append(key)
            ntok.append(int(r["input_lengths"]))
            groups.append(grp)
        return BatchMeta(partition, keys, ntok, groups, set(ROLLOUT_FIELDS)), metrics

    def shutdown(self) -> None:
        self.generation.finish_generation()


class PlanePolicy:
    """The policy seen through the data plane: every call takes a :class:`BatchMeta`, the ranks fetch their own samples,
    and per-token results go back to the plane instead of to the caller."""

    def __init__(self, policy, plane: DataPlaneClient, pad_token_id: int = 0, dp_cfg: Optional[dict] = None):
        self.policy, self.plane, self.pad = policy, plane, pad_token_id
        self.dp_cfg = dict(dp_cfg or {"enabled": True})
        self._step: Optional[dict] = None

    def __getattr__(self, name):           # everything else (prepare_for_training, save_checkpoint, ...) is the worker's
        return getattr(self.policy, name)

    # ---- partition lifecycle
    def prepare_step(self, partition: str) -> str:
        stale = [m.key for m in self.plane.list_meta(partition + "/")]
        if stale:
            self.plane.delete(stale)
        return partition

    def discard_samples(self, keys: Sequence[str]) -> None:
        self.plane.delete(list(keys))

    def finish_step(self, meta: BatchMeta) -> None:
        self.plane.delete(meta.keys)

    # ---- IO
    def read_from_dataplane(self, meta: BatchMeta, fields: Iterable[str]) -> BatchedDataDict:
        return records_to_batch(self.plane.get(meta.keys, tuple(fields)), pad_values={"input_ids": self.pad, "prompt_ids": self.pad})

    def write_to_dataplane(self, meta: BatchMeta, fields: dict[str, Any], lengths: Optional[torch.Tensor] = None) -> None:
        for i, k in enumerate(meta.keys):
            rec: dict[str, Any] = {"__jagged__": list(JAGGED)}
            for f, v in fields.items():
                row = v[i]
                cut = lengths is not None and f in JAGGED and hasattr(row, "dim") and row.dim() >= 1
                rec[f] = row[: int(lengths[i])].clone() if cut else (row.clone() if hasattr(row, "clone") else row)
            self.plane.update(k, rec)
        meta.fields |= set(fields)

    # ---- compute
    def _fetch(self, meta: BatchMeta, fields: Iterable[str]) -> BatchedDataDict:
        return fetch_batch(self.plane, meta.keys, tuple(fields), pad_values={"input_ids": self.pad})

    def get_logprobs_from_meta(self, meta: BatchMeta, out_field: str = "prev_logprobs") -> None:
        data = self._fetch(meta, ("input_ids", "input_lengths"))
        lp = self.policy.get_logprobs(data)["logprobs"]
        self.write_to_dataplane(meta, {out_field: lp}, lengths=data["input_lengths"])

    def get_reference_policy_logprobs_from_meta(self, meta: BatchMeta, out_field: str = "reference_policy_logprobs") -> None:
        data = self._fetch(meta, ("input_ids", "input_lengths"))
        lp = self.policy.get_reference_policy_logprobs(data)["reference_logprobs"]
        self.write_to_dataplane(meta, {out_field: lp}, lengths=data["input_lengths"])

    def train_from_meta(self, meta: BatchMeta, loss_fn, gbs: Optional[int] = None, mbs: Optional[int] = None,
                        fields: Iterable[str] = TRAIN_FIELDS) -> dict:
        data = self._fetch(meta, [f for f in fields if f in meta.fields])
        return self.policy.train(data, loss_fn, gbs=gbs, mbs=mbs)

    # ---- a training step fed in several pieces (streaming micro-batches while later rollouts still arrive)
    def begin_train_step(self, loss_fn, gbs: Optional[int] = None, mbs: Optional[int] = None) -> None:
        assert self._step is None, "a training step is already open"
        self._step = dict(loss_fn=loss_fn, gbs=gbs, mbs=mbs, metas=[])

    def train_microbatches_from_meta(self, meta: BatchMeta) -> None:
        assert self._step is not None, "begin_train_step first"
        self._step["metas"].append(meta)

    def finish_train_step(self) -> dict:
        """Runs the optimizer step over everything queued since ``begin_train_step`` (one global batch)."""
        st, self._step = self._step, None
        assert st is not None and st["metas"], "nothing to train on"
        m0 = st["metas"][0]
        merged = BatchMeta(m0.partition, [k for m in st["metas"] for k in m.keys], [n for m in st["metas"] for n in m.num_tokens],
                           [g for m in st["metas"] for g in m.groups], set.intersection(*[set(m.fields) for m in st["metas"]]))
        return self.train_from_meta(merged, st["loss_fn"], gbs=st["gbs"] or merged.size * max(1, _world()[1]), mbs=st["mbs"])

    def abort_train_step(self) -> None:
        self._step = None


def _seq_logprob_error(data: BatchedDataDict) -> dict:
    """exp(mean |log p_train - log p_gen|) over generated tokens: the engine / trainer mismatch gate of the reference."""
    m = data["token_mask"][:, 1:].float() * data["sample_mask"].float()[:, None]
    a, b = data["prev_logprobs"][:, 1:], data["generation_logprobs"][:, 1:]
    n = m.sum().clamp(min=1)
    err = ((a - b).abs() * m).sum() / n
    return {"token_mult_prob_error": float(torch.exp(err))}


def grpo_train_sync(policy, generation, dataloader, val_dataloader, tokenizer, loss_fn, task_to_env, val_task_to_env, logger,
                    checkpointer, save_state: dict, master_config: dict, data_plane: Optional[DataPlaneClient] = None,
                    step_callback: Optional[Callable[[int, dict], None]] = None) -> dict:
    """GRPO whose training data lives in the data plane between rollout and optimizer step. Same arguments as
    ``grpo_train`` plus the data-plane client (created from ``master_config['data_plane']`` when absent)."""
    cfg = master_config
    dp_cfg = cfg.get("data_plane") or {}
    if data_plane is None:
        if not dp_cfg.get("enabled", False):
            raise ValueError("grpo_train_sync needs data_plane.enabled = true (use grpo_train for the in-memory path)")
        from rl_b200.data_plane import create_data_plane

        data_plane = create_data_plane(dp_cfg)
    rank, world = _world()
    g, pcfg = cfg["grpo"], cfg["policy"]
    loss_cfg = cfg.get("loss_fn") or {}
    timer = Timer()
    pad = tokenizer.pad_token_id if tokenizer is not None and tokenizer.pad_token_id is not None else 0
    adv = create_advantage_estimator(g, loss_cfg)
    pol = policy if isinstance(policy, PlanePolicy) else PlanePolicy(policy, data_plane, pad, dp_cfg)
    actor = SyncRolloutActor(pol.policy, generation, tokenizer, task_to_env, cfg, data_plane, timer)
    use_ref = loss_fn.cfg["reference_policy_kl_penalty"] != 0 and not g.get("skip_reference_policy_logprobs_calculation", False) \
        and getattr(pol.policy, "ref_flat", None) is not None
    total_steps = save_state.get("total_steps", 0)
    last: dict = {}
    stale = True
    for batch in dataloader:
        if total_steps >= g["max_num_steps"]:
            break
        part = pol.prepare_step(f"train/{total_steps:08d}")
        with timer.time("total_step_time"):
            with timer.time("prepare_for_generation"):
                if stale:
                    refit_policy_generation(pol.policy, generation, timer)
                    stale = False
            meta, gen_metrics = actor.rollout_to_plane(batch, part, weight_version=total_steps)
            generation.finish_generation()
            # ---- the driver touches only the small fields
            with timer.time("reward_calculation"):
                small = pol.read_from_dataplane(meta, DRIVER_FIELDS)
                rewards = small["total_reward"].float()
                advantages = adv.compute_advantage(small["prompt_ids"], rewards, small["token_mask"], valid_mask=torch.ones_like(rewards))
                pol.write_to_dataplane(meta, {"advantages": advantages}, lengths=small["input_lengths"])
            with timer.time("policy_and_reference_logprobs"):
                pol.prepare_for_lp_inference()
                pol.get_logprobs_from_meta(meta)
                if use_ref:
                    pol.get_reference_policy_logprobs_from_meta(meta)
                else:
                    z = torch.zeros_like(advantages)
                    pol.write_to_dataplane(meta, {"reference_policy_logprobs": z}, lengths=small["input_lengths"])
            err = _seq_logprob_error(pol.read_from_dataplane(meta, ("prev_logprobs", "generation_logprobs", "token_mask", "sample_mask")))
            with timer.time("policy_training"):
                pol.prepare_for_training()
                res = pol.train_from_meta(meta, loss_fn, gbs=pcfg["train_global_batch_size"], mbs=pcfg["train_micro_batch_size"])
                stale = True
            plane_stats = data_plane.stats()
            pol.finish_step(meta)
        total_steps += 1
        metrics = _aggregate_train_metrics(res)
        metrics.update(reward=float(rewards.mean()), samples=float(meta.size), **err)
        metrics["data_plane_resident_after_step"] = float(data_plane.stats().get("resident_samples", 0))
        metrics["data_plane_resident_peak"] = float(plane_stats.get("resident_samples", 0))
        save_state.update(total_steps=total_steps, current_step=total_steps)
        if logger is not None:
            logger.log_metrics(metrics, total_steps, prefix="train")
            logger.log_metrics(timer.get_timing_metrics("sum"), total_steps, prefix="timing/train")
        if _is_main():
            print(f"[grpo_sync] step {total_steps}: loss={metrics['loss']:.5f} reward={metrics['reward']:.4f} "
                  f"mult_prob_err={err['token_mult_prob_error']:.4f}", flush=True)
        last = {"train": metrics, "generation": gen_metrics, "timing": timer.get_timing_metrics("sum")}
        if step_callback is not None:
            step_callback(total_steps, last)
        ck = cfg.get("checkpointing") or {}
        if checkpointer is not None and getattr(checkpointer, "enabled", False) and ck.get("save_period") and total_steps % ck["save_period"] == 0:
            from rl_b200.algorithms.grpo import save_checkpoint

            save_checkpoint(pol.policy, dataloader, checkpointer, save_state, cfg, total_steps)
        timer.reset()
    return last
