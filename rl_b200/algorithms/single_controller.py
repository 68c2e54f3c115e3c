"""Single-controller GRPO over the data plane.

One long-lived controller owns two pumps: the *rollout pump* turns prompts into trajectories and stores them, sample by
sample, in the data plane, tagged with the weight version that produced them; the *train pump* picks complete prompt
groups that are young enough, fetches them by key, writes log-probabilities and advantages back, trains and publishes a
new weight version. A stall watchdog observes both pumps, a health tracker the generation side; the controller can be
checkpointed between steps. The structure follows nemo_rl/algorithms/single_controller.py:92-1607 (pumps :445 / :843,
watchdog :1223, fleet probe :1311, checkpoint :1513, weight sync :1607).

Trainer and engine share the GPU in this runtime, so the pumps take turns on it (``engine_lock``); with
``pump_mode="threads"`` they are real threads and host work (environments, tokenisation, data-plane traffic) of one
overlaps device work of the other; ``pump_mode="interleaved"`` runs the same pumps from one thread in a fixed order,
which multi-rank jobs need because every rank must enter its collectives in the same order.
"""

from __future__ import annotations

import threading
import time
from typing import Callable, Optional

import torch

from rl_b200.algorithms.advantage_estimator import create_advantage_estimator
from rl_b200.algorithms.async_grpo import _collect
from rl_b200.algorithms.grpo import _aggregate_train_metrics, _is_main, build_train_data, refit_policy_generation
from rl_b200.data_plane import LocalDataPlane, SampleMeta, preshard
from rl_b200.data_plane.codec import batch_to_records, records_to_batch
from rl_b200.distributed.health import HealthPolicy, HealthTracker, ShardState, StallWatchdog
from rl_b200.utils.timer import Timer

SC_DEFAULTS = dict(max_trajectory_age_steps=1, rollout_ahead_batches=2, pump_mode="interleaved", stall_timeout_s=600.0,
                   max_generation_failures=3, poll_s=0.01, probe_interval_s=30.0, probe_prompt_tokens=4, restart_dead_engine=True)


class ControllerStalled(RuntimeError):
    pass


class SingleController:
    def __init__(self, policy, generation, dataloader, tokenizer, loss_fn, task_to_env, cfg: dict, data_plane=None, logger=None,
                 checkpointer=None, save_state: Optional[dict] = None, step_callback: Optional[Callable] = None):
        self.policy, self.generation, self.tokenizer, self.loss_fn, self.envs = policy, generation, tokenizer, loss_fn, task_to_env
        self.cfg, self.logger, self.checkpointer, self.step_callback = cfg, logger, checkpointer, step_callback
        self.g, self.pcfg = cfg["grpo"], cfg["policy"]
        sc = dict(SC_DEFAULTS)
        sc.update(cfg.get("single_controller") or {})
        self.sc = sc
        self.plane = data_plane or LocalDataPlane()
        self.save_state = save_state if save_state is not None else {"total_steps": 0, "weight_version": 0}
        self.version = int(self.save_state.get("weight_version", 0))
        self.steps = int(self.save_state.get("total_steps", 0))
        self.pad = tokenizer.pad_token_id if tokenizer is not None and tokenizer.pad_token_id is not None else 0
        self.adv = create_advantage_estimator(self.g, cfg.get("loss_fn") or {})
        self.timer = Timer()
        self._data_iter = iter(dataloader)
        self._exhausted = False
        self._batch_seq = 0
        self._refit_needed = True
        self.engine_lock = threading.Lock()
        self._stop = threading.Event()
        self._error: Optional[BaseException] = None
        self.health = HealthTracker(1, HealthPolicy(dead_after_failures=int(sc["max_generation_failures"])))
        self.watchdog = StallWatchdog(float(sc["stall_timeout_s"]), on_stall=self._on_stall)
        self.stats = dict(rollout_batches=0, samples_stored=0, samples_trained=0, dropped_stale=0, generation_failures=0,
                          weight_syncs=0, weight_sync_s=0.0, probes=0, probe_failures=0, engine_restarts=0)
        self.engine_version = -1           # the weight version the engine serves (set by the weight-sync pump)
        self._last_probe = time.monotonic()
        self.use_ref = loss_fn.cfg["reference_policy_kl_penalty"] != 0 and policy.ref_flat is not None
        assert loss_fn.cfg["use_importance_sampling_correction"] or int(sc["max_trajectory_age_steps"]) == 0, \
            "off-policy trajectories need loss_fn.use_importance_sampling_correction=true"

    # ------------------------------------------------------------------ rollout pump
    def _pending_batches(self) -> int:
        return len({m.extra.get("batch") for m in self.plane.list_meta("done/")})

    def rollout_once(self) -> int:
        """One prompt batch -> trajectories -> data plane. Returns the number of samples stored (0: nothing to do)."""
        if self._exhausted or self.health.state(0) in (ShardState.DEAD, ShardState.RETIRED):
            return 0
        try:
            batch = next(self._data_iter)
        except StopIteration:
            self._exhausted = True
            return 0
        with self.engine_lock:
            try:
                self._sync_weights_locked()      # (no-op when the weight-sync pump already brought the engine up to date)
                version = self.engine_version
                traj, _ = _collect(self.policy, self.generation, batch, self.tokenizer, self.envs, self.cfg, self.pad, self.timer)
                self.generation.finish_generation()
                self.health.report_success(0)
            except Exception as e:   # an engine failure costs this batch, not the controller
                self.stats["generation_failures"] += 1
                if self.health.report_failure(0, f"{type(e).__name__}: {e}") == ShardState.DEAD:
                    raise
                return 0
        td = build_train_data(traj, self.pad)
        td["total_reward"] = traj["total_reward"].float()
        td["prompt_ids"] = traj["_prompt_ids"]
        td["prompt_idx"] = traj["idx"]
        recs = batch_to_records(td, jagged=("input_ids", "token_mask", "generation_logprobs"))
        b = self._batch_seq
        self._batch_seq += 1
        for i, r in enumerate(recs):
            key = f"traj/{b:08d}/{i:05d}"
            self.plane.put(key, r, SampleMeta(key, num_tokens=int(r["input_lengths"]), weight_version=version,
                                              group=f"{b}:{int(r['prompt_idx'])}", extra={"batch": b}))
        # the batch becomes visible to the train pump only now that every sample of it is stored
        self.plane.put(f"done/{b:08d}", {"n": len(recs)}, SampleMeta(f"done/{b:08d}", weight_version=version, extra={"batch": b}))
        self.stats["rollout_batches"] += 1
        self.stats["samples_stored"] += len(recs)
        self.watchdog.progress()
        return len(recs)

    # ------------------------------------------------------------------ weight-sync pump
    def _sync_weights_locked(self) -> bool:
        if not self._refit_needed and self.engine_version == self.version:
            return False
        t0 = time.perf_counter()
        refit_policy_generation(self.policy, self.generation, self.timer)
        self._refit_needed = False
        self.engine_version = self.version
        self.stats["weight_syncs"] += 1
        self.stats["weight_sync_s"] += time.perf_counter() - t0
        return True

    def sync_weights_once(self, blocking: bool = False) -> bool:
        """Brings the engine to the trainer's current weight version as soon as the engine is free, instead of at the start of
        the next rollout: the rollout pump then finds a current engine and generation starts without the refit in front of it
        (role of the controller's weight-sync pump, nemo_rl/algorithms/single_controller.py:1607). Returns whether it synced."""
        if not self._refit_needed and self.engine_version == self.version:
            return False
        if not self.engine_lock.acquire(blocking=blocking):
            return False
        try:
            return self._sync_weights_locked()
        except Exception as e:
            self.stats["generation_failures"] += 1
            self.health.report_failure(0, f"weight sync: {type(e).__name__}: {e}")
            return False
        finally:
            self.engine_lock.release()

    # ------------------------------------------------------------------ fleet probe pump
    def probe_once(self, force: bool = False) -> Optional[bool]:
        """A cheap liveness check of the generation side between rollouts (a few tokens through the engine, or the engine's own
        ``health_check`` when it has one): failures feed the same health tracker the rollouts report to, so a dead engine is
        found before a whole prompt batch is spent on it, and is restarted (``generation.restart()`` when available, else
        sleep / wake) when ``restart_dead_engine`` (nemo_rl/algorithms/single_controller.py:1311). None: not due, or busy."""
        now = time.monotonic()
        if not force and now - self._last_probe < float(self.sc["probe_interval_s"]):
            return None
        if not self.engine_lock.acquire(blocking=False):
            return None
        try:
            self._last_probe = now
            self.stats["probes"] += 1
            try:
                hc = getattr(self.generation, "health_check", None)
                if hc is not None:
                    ok = bool(hc())
                else:
                    from rl_b200.distributed.batched_data_dict import BatchedDataDict

                    n = int(self.sc["probe_prompt_tokens"])
                    self._sync_weights_locked()
                    out = self.generation.generate(BatchedDataDict(input_ids=torch.full((1, n), max(self.pad - 1, 0), dtype=torch.long),
                                                                   input_lengths=torch.tensor([n])), greedy=True)
                    self.generation.finish_generation()
                    ok = int(out["generation_lengths"][0]) > 0
                if not ok:
                    raise RuntimeError("the engine answered the probe with nothing")
                self.health.report_success(0)
                return True
            except Exception as e:
                self.stats["probe_failures"] += 1
                state = self.health.report_failure(0, f"probe: {type(e).__name__}: {e}")
                if state == ShardState.DEAD and self.sc["restart_dead_engine"]:
                    self._restart_engine()
                return False
        finally:
            self.engine_lock.release()

    def _restart_engine(self) -> None:
        if self.health.begin_restart(0) != ShardState.RESTARTING:      # restart budget spent: the shard is retired
            return
        ok = True
        try:
            if hasattr(self.generation, "restart"):
                self.generation.restart()
            else:
                self.generation.shutdown()
                self.generation.prepare_for_generation()
            self._refit_needed = True
            self.engine_version = -1
            self.stats["engine_restarts"] += 1
        except Exception:
            ok = False
        self.health.finish_restart(0, ok, weight_version=self.health.current_weight_version)

    # ------------------------------------------------------------------ train pump
    def _select(self) -> Optional[list[SampleMeta]]:
        """The oldest stored batch that is young enough; batches that aged out are deleted."""
        max_age = int(self.sc["max_trajectory_age_steps"])
        by_batch: dict[int, list[SampleMeta]] = {}
        done = {m.extra.get("batch") for m in self.plane.list_meta("done/")}
        for m in self.plane.list_meta("traj/"):
            if m.extra.get("batch") in done:
                by_batch.setdefault(m.extra.get("batch"), []).append(m)
        for b in sorted(by_batch):
            ms = by_batch[b]
            if self.version - min(m.weight_version for m in ms) > max_age:
                self.stats["dropped_stale"] += self.plane.delete([m.key for m in ms])
                self.plane.delete([f"done/{b:08d}"])
                continue
            return sorted(ms, key=lambda m: m.key)
        return None

    def train_once(self) -> Optional[dict]:
        metas = self._select()
        if metas is None:
            return None
        keys = preshard(metas, 1)[0]
        order = {m.key: m for m in metas}
        keys = sorted(keys)
        data = records_to_batch(self.plane.get(keys, ("input_ids", "input_lengths", "token_mask", "sample_mask", "generation_logprobs",
                                                       "total_reward", "prompt_ids")),
                                pad_values={"input_ids": self.pad})
        pid = data["prompt_ids"]   # one stored batch came from one prompt batch: equal padded width
        rewards = data["total_reward"].float()
        with self.engine_lock:
            with self.timer.time("policy_and_reference_logprobs"):
                self.policy.prepare_for_lp_inference()
                data["prev_logprobs"] = self.policy.get_logprobs(data)["logprobs"]
                data["reference_policy_logprobs"] = (self.policy.get_reference_policy_logprobs(data)["reference_logprobs"]
                                                     if self.use_ref else torch.zeros_like(data["prev_logprobs"]))
            data["advantages"] = self.adv.compute_advantage(pid, rewards, data["token_mask"], valid_mask=torch.ones_like(rewards))
            with self.timer.time("policy_training"):
                self.policy.prepare_for_training()
                res = self.policy.train(data, self.loss_fn, gbs=self.pcfg["train_global_batch_size"], mbs=self.pcfg["train_micro_batch_size"])
            self.version += 1
            self._refit_needed = True
        age = self.version - 1 - min(order[k].weight_version for k in keys)
        self.plane.delete(keys)
        self.plane.delete([f"done/{order[keys[0]].extra.get('batch'):08d}"])
        self.steps += 1
        self.stats["samples_trained"] += len(keys)
        metrics = _aggregate_train_metrics(res)
        metrics.update(reward=float(rewards.mean()), trajectory_age=float(age), weight_version=float(self.version),
                       engine_version=float(self.engine_version), weight_syncs=float(self.stats["weight_syncs"]),
                       stored_samples=float(self.plane.stats().get("resident_samples", 0)))
        self.save_state.update(total_steps=self.steps, current_step=self.steps, weight_version=self.version)
        if self.logger is not None:
            self.logger.log_metrics(metrics, self.steps, prefix="train")
        if _is_main():
            print(f"[single_controller] step {self.steps}: loss={metrics['loss']:.5f} reward={metrics['reward']:.4f} age={age} "
                  f"stored={int(metrics['stored_samples'])}", flush=True)
        self.watchdog.progress()
        out = {"train": metrics, "timing": self.timer.get_timing_metrics("sum")}
        if self.step_callback is not None:
            self.step_callback(self.steps, out)
        self.timer.reset()
        return out

    # ------------------------------------------------------------------ supervision
    def _on_stall(self, idle_s: float) -> None:
        self._error = ControllerStalled(f"no rollout or training progress for {idle_s:.0f} s")
        self._stop.set()

    def state_dict(self) -> dict:
        """Everything needed to resume: counters and the keys still stored (their payload lives in the data plane)."""
        return dict(version=self.version, steps=self.steps, batch_seq=self._batch_seq, stats=dict(self.stats),
                    pending=[(m.key, m.weight_version, m.group) for m in self.plane.list_meta("traj/")])

    def load_state_dict(self, sd: dict) -> None:
        self.version, self.steps, self._batch_seq = sd["version"], sd["steps"], sd["batch_seq"]
        self.stats.update(sd.get("stats", {}))
        self._refit_needed = True

    # ------------------------------------------------------------------ run
    def run(self, max_steps: Optional[int] = None) -> dict:
        max_steps = max_steps if max_steps is not None else self.g["max_num_steps"]
        ahead = int(self.sc["rollout_ahead_batches"])
        last: dict = {}
        self.watchdog.start()
        try:
            if self.sc["pump_mode"] == "threads":
                def pump():
                    try:
                        while not self._stop.is_set():
                            if self._pending_batches() >= ahead or self.rollout_once() == 0:
                                if self._exhausted:
                                    return
                                time.sleep(float(self.sc["poll_s"]))
                    except BaseException as e:
                        self._error = e
                        self._stop.set()

                def side_pumps():     # weight sync as soon as the engine is free; a health probe every probe_interval_s
                    while not self._stop.is_set():
                        try:
                            self.sync_weights_once()
                            self.probe_once()
                        except BaseException as e:
                            self._error = e
                            self._stop.set()
                        time.sleep(float(self.sc["poll_s"]))

                t = threading.Thread(target=pump, daemon=True, name="rlb-rollout-pump")
                t.start()
                threading.Thread(target=side_pumps, daemon=True, name="rlb-sync-probe-pumps").start()
                while self.steps < max_steps and not self._stop.is_set():
                    out = self.train_once()
                    if out is None:
                        if self._exhausted and not t.is_alive() and self._select() is None:
                            break
                        time.sleep(float(self.sc["poll_s"]))
                    else:
                        last = out
                self._stop.set()
                t.join(60)
            else:
                while self.steps < max_steps and not self._stop.is_set():
                    while self._pending_batches() < ahead and self.rollout_once() > 0:
                        pass
                    out = self.train_once()
                    self.sync_weights_once(blocking=True)
                    self.probe_once()
                    if out is None:
                        if self._exhausted:
                            break
                        continue
                    last = out
        finally:
            self.watchdog.stop()
        if self._error is not None:
            raise self._error
        return last
