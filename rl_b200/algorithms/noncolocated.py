"""Asynchronous GRPO on split GPU sets: generation ranks produce trajectories while training ranks train, at the same
time, on different GPUs.

Job layout (``rl_b200/distributed/roles.py``): the first T ranks train (their default process group holds only them),
the last G ranks each run a generation engine with a complete copy of the weights. Three channels connect the sets:

  * trajectories: a generation rank writes the finished rollouts of one *shard* (the prompts of one training rank for one
    step, already scored by the environments) into the job's TCP store; the training rank that owns the shard reads it.
    Shard s = step * T + trainer rank is produced by generation rank s mod G, so every rank knows its work without a
    dispatcher;
  * weights: after an optimizer step training rank 0 announces a new version in the store and broadcasts the HF-named
    tensors in packed buckets over the sync communicator; generation ranks join the broadcast at their next poll point
    (between two ``generate`` calls, or between two decode windows with ``in_flight_weight_updates``);
  * control: completed training steps, the stop flag.

Staleness is bounded by construction: a generation rank starts shard (step, .) only while ``step <= completed + max_age``
and with weights of version ``>= step - max_age``, so every trajectory that reaches the loss is at most
``max_trajectory_age_steps`` versions old; the loss then needs ``use_importance_sampling_correction`` as for any
off-policy sample. This is the overlap of nemo_rl/algorithms/grpo.py:4074-5462 (background trajectory collector
``async_utils/trajectory_collector.py:76``, replay buffer ``async_utils/replay_buffer.py:40``) without a Ray driver.
"""

from __future__ import annotations

import io
import pickle
import time
from typing import Callable, Optional

import torch

from rl_b200.algorithms.advantage_estimator import create_advantage_estimator
from rl_b200.distributed.batched_data_dict import BatchedDataDict
from rl_b200.distributed.roles import RoleLayout, SyncGroup
from rl_b200.utils.timer import Timer

_CHUNK = 4 << 20
DEFAULT_BUCKET_BYTES = 256 << 20


# ------------------------------------------------------------------------------------------------ store channels
class Control:
    """Counters and flags of the job in the TCP store."""

    def __init__(self, store):
        self.store = store

    def completed_steps(self) -> int:
        return int(self.store.add("ctl/train_steps", 0))

    def step_done(self) -> int:
        return int(self.store.add("ctl/train_steps", 1))

    def announce_weights(self, version: int) -> None:
        self.store.set("ctl/weights_pending", str(version))

    def pending_weights(self) -> int:
        if not self.store.check(["ctl/weights_pending"]):
            return 0
        return int(bytes(self.store.get("ctl/weights_pending")).decode())

    def stop(self) -> None:
        self.store.set("ctl/stop", "1")

    def stopped(self) -> bool:
        return bool(self.store.check(["ctl/stop"]))


class TrajectoryChannel:
    """Shards of finished rollouts, keyed by (step, trainer rank), in the job store."""

    def __init__(self, store):
        self.store = store

    @staticmethod
    def _key(step: int, trainer_rank: int) -> str:
        return f"traj/{step}/{trainer_rank}"

    def push(self, step: int, trainer_rank: int, batch: BatchedDataDict, weight_version: int, gen_seconds: float) -> int:
        buf = io.BytesIO()
        torch.save({"batch": dict(batch), "weight_version": weight_version, "gen_seconds": gen_seconds}, buf)
        raw = buf.getvalue()
        k = self._key(step, trainer_rank)
        n = max(1, -(-len(raw) // _CHUNK))
        for i in range(n):
            self.store.set(f"{k}/c{i}", raw[i * _CHUNK : (i + 1) * _CHUNK])
        self.store.set(f"{k}/n", str(n))     # written last: its presence means the shard is complete
        return len(raw)

    def pop(self, step: int, trainer_rank: int, ctl: Control, poll_s: float = 0.002, timeout_s: float = 3600.0) -> Optional[dict]:
        k = self._key(step, trainer_rank)
        t0 = time.time()
        while not self.store.check([f"{k}/n"]):
            if ctl.stopped():
                return None
            if time.time() - t0 > timeout_s:
                raise TimeoutError(f"no trajectories for step {step} / trainer rank {trainer_rank} after {timeout_s:.0f} s")
            time.sleep(poll_s)
        n = int(bytes(self.store.get(f"{k}/n")).decode())
        raw = b"".join(bytes(self.store.get(f"{k}/c{i}")) for i in range(n))
        for i in range(n):
            self.store.delete_key(f"{k}/c{i}")
        self.store.delete_key(f"{k}/n")
        item = torch.load(io.BytesIO(raw), weights_only=False)
        item["batch"] = BatchedDataDict(item["batch"])
        item["wait_seconds"] = time.time() - t0
        return item


# ------------------------------------------------------------------------------------------------ weights
def _buckets(items, bucket_bytes: int):
    cur, size = [], 0
    for name, t in items:
        nb = t.numel() * t.element_size()
        if cur and size + nb > bucket_bytes:
            yield cur
            cur, size = [], 0
        cur.append((name, t))
        size += nb
    if cur:
        yield cur


def publish_weights(policy, sync: Optional[SyncGroup], ctl: Control, version: int, bucket_bytes: int = DEFAULT_BUCKET_BYTES) -> int:
    """Training side. Collective over the tensor-parallel group of training rank 0 (full tensors are assembled there);
    only the rank that owns ``sync`` announces the version and sends. Returns the payload bytes."""
    from rl_b200.models.hf_io import iter_hf_tensors
    from rl_b200.refit.packed_broadcast import pack

    total = 0
    if sync is not None:
        ctl.announce_weights(version)
    for bucket in _buckets(((n, t.detach()) for n, t in iter_hf_tensors(policy.model)), bucket_bytes):
        if sync is None:
            continue   # a tensor-parallel peer of rank 0: it only takes part in assembling the tensors
        meta = [(n, tuple(t.shape), t.dtype) for n, t in bucket]
        sync.broadcast_object(("bucket", version, meta), 0)
        buf = pack([t for _, t in bucket], sync.device)
        sync.broadcast_tensor(buf, 0)
        total += buf.numel()
    if sync is not None:
        sync.broadcast_object(("end", version, None), 0)
    return total


class WeightReceiver:
    """Generation side: joins the trainer's broadcast when a newer version has been announced."""

    def __init__(self, model, sync: SyncGroup, ctl: Control):
        from rl_b200.models.hf_io import iter_hf_shards

        self.model, self.sync, self.ctl = model, sync, ctl
        self.version = 0
        self._dst = {hf: (dst, hs) for hf, dst, hs in iter_hf_shards(model)}
        self.updates = 0
        self.bytes = 0

    @torch.no_grad()
    def poll(self) -> bool:
        """Receives every announced version that this rank has not applied yet. Returns True if the weights changed."""
        from rl_b200.refit.packed_broadcast import unpack

        changed = False
        while self.ctl.pending_weights() > self.version:
            while True:
                kind, version, meta = self.sync.broadcast_object(None, 0)
                if kind == "end":
                    self.version = version
                    break
                size = sum(-(-_numel(s) * torch.empty((), dtype=d).element_size() // 16) * 16 for _, s, d in meta)
                buf = torch.empty(size, dtype=torch.uint8, device=self.sync.device)
                self.sync.broadcast_tensor(buf, 0)
                self.bytes += size
                for name, t in unpack(buf, meta):
                    hit = self._dst.get(name)
                    if hit is None:
                        continue
                    dst, hs = hit
                    dst.copy_((t if hs is None else t.narrow(hs[0], hs[1], hs[2])).to(dst.dtype))
            self.updates += 1
            changed = True
        return changed


def _numel(shape) -> int:
    n = 1
    for s in shape:
        n *= s
    return n


# ------------------------------------------------------------------------------------------------ generation ranks
def build_generation_rank(cfg: dict, tokenizer, model_cfg=None, device=None):
    """The model and engine of a generation rank: the policy's architecture with uninitialised weights (the trainer's
    first broadcast fills them) behind the ordinary generation facade."""
    from rl_b200.engine.generation import NativeGeneration
    from rl_b200.models.config import ModelConfig, preset
    from rl_b200.models.transformer import build_model

    pcfg = cfg["policy"]
    if model_cfg is None:
        name = pcfg.get("model_name")
        from rl_b200.models.config import PRESETS

        model_cfg = preset(name, **(pcfg.get("hf_config_overrides") or {})) if name in PRESETS else ModelConfig.from_pretrained(name)
    device = device or (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
    dtype = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
             "float16": torch.float16}[pcfg.get("precision", "bfloat16")]
    model = build_model(model_cfg, dtype=dtype, device=device, seed=0)
    g = dict(pcfg.get("generation") or {})
    native_cfg = dict(g.get("native_cfg") or g.get("vllm_cfg") or {})
    merged = {k: v for k, v in g.items() if k not in ("native_cfg", "vllm_cfg", "colocated", "sglang_cfg")}
    for k in ("gpu_memory_utilization", "max_model_len", "block_size", "kv_cache_tokens", "max_running", "use_cuda_graphs", "decode_window"):
        if k in native_cfg:
            merged[k] = native_cfg[k]
    merged.setdefault("max_model_len", pcfg["max_total_sequence_length"])
    return NativeGeneration(model, merged, tokenizer)


def generation_service(layout: RoleLayout, cfg: dict, generation, dataset, tokenizer, task_to_env: dict, collate_fn=None,
                       step_callback: Optional[Callable] = None) -> dict:
    """Main loop of a generation rank: produce the shards assigned to this rank, within the staleness bound, with the
    newest weights; leave when the trainers raise the stop flag. Returns counters (shards, tokens, weight updates)."""
    from rl_b200.algorithms.async_grpo import ASYNC_DEFAULTS, _collect
    from rl_b200.algorithms.grpo import GRPO_DEFAULTS, _ShardedPromptLoader
    from rl_b200.data.collate import rl_collate_fn

    g = dict(GRPO_DEFAULTS)
    g.update(cfg.get("grpo") or {})
    cfg = dict(cfg, grpo=g)
    a = dict(ASYNC_DEFAULTS)
    a.update(g.get("async_grpo") or {})
    max_age = int(a["max_trajectory_age_steps"])
    T, G, me = layout.train_world, layout.gen_world, layout.role_rank
    ctl, chan = Control(layout.store), TrajectoryChannel(layout.store)
    sync = SyncGroup(layout)
    model = generation.engine.model
    recv = WeightReceiver(model, sync, ctl)
    if a.get("in_flight_weight_updates"):
        # poll between decode windows: in-flight requests continue on the new weights (their cached keys / values stay)
        generation.engine.window_hook = lambda: recv.poll() and generation.engine.requantize()
    pad = tokenizer.pad_token_id if tokenizer is not None and tokenizer.pad_token_id is not None else 0
    shuffle = bool((cfg.get("data") or {}).get("shuffle", True))
    loaders = [iter(_ShardedPromptLoader(dataset, g["num_prompts_per_step"], collate_fn or rl_collate_fn, shuffle, g["seed"], t, T)) for t in range(T)]
    timer = Timer()
    stats = dict(shards=0, generated_tokens=0, waited_s=0.0, bytes_pushed=0)
    step = 0
    while step < g["max_num_steps"] and not ctl.stopped():
        mine = [t for t in range(T) if (step * T + t) % G == me]
        batches = {}
        try:
            for t in range(T):     # every loader advances once per step so that all ranks agree on the data order
                b = next(loaders[t])
                if t in mine:
                    batches[t] = b
        except StopIteration:
            break
        for t in mine:
            # staleness bound: not further ahead than max_age steps, and with weights no older than step - max_age
            t0 = time.time()
            while not ctl.stopped():
                recv.poll()
                # versions count from 1 (the trainer's initial weights): step s is on-policy with version s + 1
                if step <= ctl.completed_steps() + max_age and recv.version >= max(1, step - max_age + 1):
                    break
                time.sleep(0.002)
            stats["waited_s"] += time.time() - t0
            if ctl.stopped():
                break
            generation.prepare_for_generation()
            version = recv.version
            t1 = time.time()
            traj, _ = _collect(None, generation, batches[t], tokenizer, task_to_env, cfg, pad, timer)
            generation.finish_generation()
            stats["bytes_pushed"] += chan.push(step, t, traj, version, time.time() - t1)
            stats["shards"] += 1
            stats["generated_tokens"] += int(traj["generation_lengths"].sum()) if "generation_lengths" in traj else 0
            if step_callback is not None:
                step_callback(step, t, version)
        step += 1
    # keep answering weight broadcasts until the trainers are done, so that training rank 0 never blocks on a missing peer
    while not ctl.stopped():
        recv.poll()
        time.sleep(0.005)
    recv.poll()
    stats.update(weight_updates=recv.updates, weight_bytes=recv.bytes, final_version=recv.version)
    return stats


# ------------------------------------------------------------------------------------------------ training ranks
def noncolocated_grpo_train(policy, layout: RoleLayout, loss_fn, logger, checkpointer, save_state, cfg, tokenizer=None,
                            step_callback: Optional[Callable] = None) -> dict:
    """Main loop of a training rank: read this rank's shard of trajectories for the step, score it with the current (and
    the reference) policy, train, publish the new weights. Generation happens elsewhere, concurrently."""
    from rl_b200.algorithms.async_grpo import ASYNC_DEFAULTS
    from rl_b200.algorithms.grpo import _aggregate_train_metrics, _all_reduce_scalars, _is_main, build_train_data, save_checkpoint

    g, pcfg = cfg["grpo"], cfg["policy"]
    a = dict(ASYNC_DEFAULTS)
    a.update(g.get("async_grpo") or {})
    max_age = int(a["max_trajectory_age_steps"])
    assert loss_fn.cfg["use_importance_sampling_correction"] or max_age == 0, \
        "off-policy trajectories need loss_fn.use_importance_sampling_correction=true"
    ctl, chan = Control(layout.store), TrajectoryChannel(layout.store)
    sync = SyncGroup(layout) if layout.role_rank == 0 else None
    from rl_b200.parallel.state import get_state

    st = get_state()
    sends = layout.role_rank == 0 or (st.tp > 1 and st.dp_rank == 0 and st.pp_rank == 0)   # rank 0 and its tensor-parallel peers
    pad = tokenizer.pad_token_id if tokenizer is not None and tokenizer.pad_token_id is not None else 0
    adv_estimator = create_advantage_estimator(g, cfg.get("loss_fn") or {})
    use_ref = loss_fn.cfg["reference_policy_kl_penalty"] != 0 and policy.ref_flat is not None
    timer = Timer()
    ck = cfg.get("checkpointing") or {}
    step = save_state["total_steps"]
    version = step
    last: dict = {}
    try:
        if sends and version == 0:
            # version 0 is the initial weights: generation ranks start from the trainer's copy, not from their own init
            version = 0
            publish_weights(policy, sync, ctl, 1)   # announced as version 1 so that pollers see "newer than nothing"
            version = 1
        base = 1   # weight version of the initial weights
        while step < g["max_num_steps"]:
            with timer.time("total_step_time"):
                with timer.time("wait_for_trajectories"):
                    item = chan.pop(step, layout.role_rank, ctl)
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
                step += 1
                with timer.time("weight_publication"):
                    if sends:
                        publish_weights(policy, sync, ctl, base + step)
                if layout.role_rank == 0:
                    ctl.step_done()
            age = (base + step - 1) - int(item["weight_version"])
            metrics = _aggregate_train_metrics(res)
            c = _all_reduce_scalars({"r": float(rewards.sum()), "n": float(rewards.numel()), "age": float(age), "k": 1.0})
            metrics.update(reward=c["r"] / max(1.0, c["n"]), trajectory_age=c["age"] / max(1.0, c["k"]),
                           generation_seconds=float(item["gen_seconds"]), trajectory_wait_seconds=float(item["wait_seconds"]))
            save_state.update(current_step=step, total_steps=step, weight_version=base + step)
            if checkpointer is not None and checkpointer.enabled and ck.get("save_period") and step % ck["save_period"] == 0:
                save_checkpoint(policy, _NoLoader(), checkpointer, save_state, cfg, step)
            timing = timer.get_timing_metrics("sum")
            if logger is not None:
                logger.log_metrics(metrics, step, prefix="train")
                logger.log_metrics(timing, step, prefix="timing/train")
            if _is_main():
                print(f"[async_grpo] step {step}: loss={metrics['loss']:.5f} reward={metrics['reward']:.4f} age={metrics['trajectory_age']:.2f} "
                      f"wait={timing.get('wait_for_trajectories', 0):.2f}s train={timing.get('policy_training', 0):.2f}s "
                      f"gen(elsewhere)={metrics['generation_seconds']:.2f}s", flush=True)
            last = {"train": metrics, "timing": timing}
            if step_callback is not None:
                step_callback(step, last)
            timer.reset()
    finally:
        import torch.distributed as dist

        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.barrier()          # every training rank is done before the generation ranks are released
        if layout.role_rank == 0:
            ctl.stop()
    return last


class _NoLoader:
    """Checkpoint stand-in for the prompt loader: the data position of a split job is the step count itself."""

    def state_dict(self):
        return {}
