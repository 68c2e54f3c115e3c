"""Rollout collection: generate -> environment step -> append observation -> repeat, for a batch of message logs.

Behaviour follows nemo_rl/experience/rollouts.py (``generate_responses`` :469-551, ``calculate_rewards`` :705-837,
``run_multi_turn_rollout`` :840-1087): generation is token-in / token-out, the generated tokens and their
log-probabilities become an assistant message, environments are looked up per sample by ``task_name``, samples
leave the active set when their environment terminates them or the sequence budget is used up.

Runtime: each rank rolls out its own shard of the prompts on its own engine (SPMD); environments are in-process
objects, so no object-store hop sits between the engine and the reward.
"""

from __future__ import annotations

from typing import Any, Optional

import torch

from rl_b200.data.llm_message_utils import batched_message_log_to_flat_message, multimodal_fields
from rl_b200.distributed.batched_data_dict import BatchedDataDict
from rl_b200.environments.interfaces import EnvironmentInterface, EnvironmentReturn


def generate_responses(generation, flat_ids: torch.Tensor, input_lengths: torch.Tensor, batch: BatchedDataDict,
                       tokenizer, greedy: bool = False, stop_strings=None, multimodal: Optional[dict] = None):
    """Generates one continuation per row, appends it to every message log as an assistant message, and returns
    (batch, generated ids per sample, generation metrics)."""
    gen_in = BatchedDataDict(input_ids=flat_ids, input_lengths=input_lengths, **(multimodal or {}))
    if stop_strings is not None:
        gen_in["stop_strings"] = stop_strings
    if "rng_ids" in batch:
        gen_in["rng_ids"] = batch["rng_ids"]
    out = generation.generate(gen_in, greedy=greedy)
    out_ids, logprobs = out["output_ids"], out["logprobs"]
    gen_lens, tot_lens = out["generation_lengths"], out["unpadded_sequence_lengths"]
    generated = []
    for i in range(flat_ids.shape[0]):
        s, e = int(input_lengths[i]), int(tot_lens[i])
        toks = out_ids[i, s:e].clone()
        generated.append(toks)
        text = tokenizer.decode(toks.tolist(), skip_special_tokens=True) if tokenizer is not None else ""
        batch["message_log"][i].append({"role": "assistant", "content": text, "token_ids": toks,
                                        "generation_logprobs": logprobs[i, s:e].clone()})
    metrics = {"mean_generation_length": float(gen_lens.float().mean()) if len(gen_lens) else 0.0,
               "total_generated_tokens": int(gen_lens.sum())}
    return batch, generated, metrics, out


def calculate_rewards(batch: BatchedDataDict, task_to_env: dict[str, EnvironmentInterface]) -> EnvironmentReturn:
    """Routes every sample to the environment of its task and reassembles the results in input order."""
    n = len(batch["message_log"])
    by_task: dict[str, list[int]] = {}
    for i, t in enumerate(batch["task_name"]):
        by_task.setdefault(t, []).append(i)
    obs: list[Any] = [None] * n
    meta: list[Any] = [None] * n
    stops: list[Any] = [None] * n
    answers: list[Any] = [None] * n
    rewards: Optional[torch.Tensor] = None
    term = torch.zeros(n, dtype=torch.bool)
    for task, idx in by_task.items():
        if task not in task_to_env:
            raise KeyError(f"no environment registered for task '{task}'")
        r = task_to_env[task].step([batch["message_log"][i] for i in idx], [batch["extra_env_info"][i] for i in idx])
        if rewards is None:
            rewards = torch.zeros((n,) + tuple(r.rewards.shape[1:]), dtype=torch.float32)
        for j, i in enumerate(idx):
            obs[i], meta[i], stops[i] = r.observations[j], r.metadata[j], r.next_stop_strings[j]
            answers[i] = r.answers[j] if r.answers is not None else None
            rewards[i] = r.rewards[j]
            term[i] = bool(r.terminateds[j])
    return EnvironmentReturn(obs, meta, stops, rewards if rewards is not None else torch.zeros(0), term, answers)


def environment_metrics(batch: BatchedDataDict, task_to_env: dict[str, EnvironmentInterface]) -> dict[str, float]:
    """Every environment's own view of the finished batch (``global_post_process_and_metrics``: accuracy, properly-ended
    fraction, pass@samples...), per task: ``<task>/<metric>``, and without the prefix when the batch has one task only
    (nemo_rl/experience/rollouts.py runs the same hook after its rollouts)."""
    tasks = batch.get("task_name")
    if tasks is None or "total_reward" not in batch:
        return {}
    by_task: dict[str, list[int]] = {}
    for i, t in enumerate(tasks):
        by_task.setdefault(t, []).append(i)
    out: dict[str, float] = {}
    for task, idx in by_task.items():
        env = task_to_env.get(task)
        hook = getattr(env, "global_post_process_and_metrics", None)
        if hook is None:
            continue
        sub = batch.select_indices(idx)
        try:
            res = hook(sub)
        except Exception:      # a metrics hook must never cost the step its samples
            continue
        m = res[1] if isinstance(res, tuple) and len(res) == 2 else {}
        for k, v in (m or {}).items():
            if isinstance(v, (int, float)):
                out[f"{task}/{k}"] = float(v)
                if len(by_task) == 1:
                    out[k] = float(v)
    return out


def run_multi_turn_rollout(generation, input_batch: BatchedDataDict, tokenizer, task_to_env: dict[str, EnvironmentInterface],
                           max_seq_len: int, max_rollout_turns: int = 1, greedy: bool = False,
                           pad_token_id: int = 0) -> tuple[BatchedDataDict, dict[str, Any]]:
    """Runs up to ``max_rollout_turns`` generate/step rounds. Returns the batch (message logs extended in place,
    ``total_reward`` [B], ``truncated`` [B]) and rollout metrics."""
    batch = input_batch
    n = len(batch["message_log"])
    active = list(range(n))
    total_reward = torch.zeros(n, dtype=torch.float32)
    reward_components = None
    truncated = torch.zeros(n, dtype=torch.bool)
    gen_tokens = torch.zeros(n, dtype=torch.long)
    turns = torch.zeros(n, dtype=torch.long)
    answers: list[Any] = [None] * n
    stop_strings = batch.get("stop_strings")
    gen_metrics_acc: dict[str, float] = {"total_generated_tokens": 0}
    routed = None
    for turn in range(max_rollout_turns):
        if not active:
            break
        sub = batch.select_indices(active)
        sub["message_log"] = [batch["message_log"][i] for i in active]  # same list objects: appended in place
        flat, lens = batched_message_log_to_flat_message(sub["message_log"], {"token_ids": pad_token_id})
        ss = [stop_strings[i] for i in active] if stop_strings is not None else None
        sub, generated, gm, out = generate_responses(generation, flat["token_ids"], lens, sub, tokenizer, greedy, ss, multimodal_fields(flat))
        gen_metrics_acc["total_generated_tokens"] += gm["total_generated_tokens"]
        if "routed_experts" in out:   # the latest call's record covers the whole sequence so far (earlier turns are its prompt)
            if routed is None:
                routed = [None] * n
            for j, i in enumerate(active):
                routed[i] = out["routed_experts"][j, : int(out["unpadded_sequence_lengths"][j])].clone()
        for j, i in enumerate(active):
            gen_tokens[i] += generated[j].numel()
            turns[i] += 1
            truncated[i] = bool(out["truncated"][j])
        env_out = calculate_rewards(sub, task_to_env)
        r = env_out.rewards
        if r.dim() > 1:
            if reward_components is None:
                reward_components = torch.zeros((n, r.shape[1]), dtype=torch.float32)
            for j, i in enumerate(active):
                reward_components[i] += r[j]
            r = r.sum(-1)
        still = []
        for j, i in enumerate(active):
            total_reward[i] += r[j]
            batch["extra_env_info"][i] = env_out.metadata[j]
            if env_out.answers is not None:
                answers[i] = env_out.answers[j]
            if stop_strings is not None:
                stop_strings[i] = env_out.next_stop_strings[j]
            done = bool(env_out.terminateds[j])
            if not done and turn + 1 < max_rollout_turns:
                ob = env_out.observations[j]
                ids = tokenizer(ob["content"], add_special_tokens=False, return_tensors="pt")["input_ids"][0] if tokenizer is not None else torch.empty(0, dtype=torch.long)
                cur = sum(int(m["token_ids"].numel()) for m in batch["message_log"][i])
                if cur + ids.numel() >= max_seq_len:
                    truncated[i] = True  # no room for the observation plus another turn
                    continue
                batch["message_log"][i].append({"role": ob.get("role", "environment"), "content": ob["content"], "token_ids": ids})
                still.append(i)
        active = still
    batch["total_reward"] = total_reward
    batch["truncated"] = truncated
    batch["answers"] = answers
    batch["generation_lengths"] = gen_tokens
    if reward_components is not None:
        batch["reward_components"] = reward_components
    if routed is not None:
        batch["routed_experts"] = routed
    batch["length"] = torch.tensor([sum(int(m["token_ids"].numel()) for m in log) for log in batch["message_log"]], dtype=torch.long)
    env_metrics = environment_metrics(batch, task_to_env)
    metrics = {
        **env_metrics,
        "total_turns": int(turns.sum()),
        "avg_turns_per_sample": float(turns.float().mean()) if n else 0.0,
        "max_turns_per_sample": int(turns.max()) if n else 0,
        "natural_termination_rate": float((~truncated).float().mean()) if n else 0.0,
        "truncation_rate": float(truncated.float().mean()) if n else 0.0,
        "mean_gen_tokens_per_sample": float(gen_tokens.float().mean()) if n else 0.0,
        "total_generated_tokens": int(gen_tokens.sum()),
        "mean_total_reward": float(total_reward.mean()) if n else 0.0,
    }
    return batch, metrics


def run_async_multi_turn_rollout(frontend, input_batch: BatchedDataDict, tokenizer, task_to_env: dict[str, EnvironmentInterface],
                                 max_seq_len: int, max_rollout_turns: int = 1, sampling: Optional[dict] = None,
                                 max_concurrency: int = 256) -> tuple[BatchedDataDict, dict[str, Any]]:
    """Sample-level rollouts: every sample runs its own generate -> environment loop on a worker thread, so a sample whose
    environment is slow (a tool call, a remote verifier) or that needs more turns does not hold the others back. The engine
    sees the concurrent requests through ``frontend`` (a :class:`rl_b200.engine.http_server.BatchingFrontend`, or anything
    with ``submit(prompt_ids, sampling) -> record``), which forms the batches. Same outputs as
    :func:`run_multi_turn_rollout` (nemo_rl/experience/rollouts.py:1172, ``run_async_multi_turn_rollout``)."""
    import concurrent.futures as cf

    batch = input_batch
    n = len(batch["message_log"])
    sampling = dict(sampling or {})
    total_reward = torch.zeros(n, dtype=torch.float32)
    truncated = torch.zeros(n, dtype=torch.bool)
    gen_tokens = torch.zeros(n, dtype=torch.long)
    turns = torch.zeros(n, dtype=torch.long)
    answers: list[Any] = [None] * n

    def one(i: int) -> None:
        log = batch["message_log"][i]
        env = task_to_env[batch["task_name"][i]]
        meta = batch["extra_env_info"][i]
        for turn in range(max_rollout_turns):
            prompt = torch.cat([m["token_ids"] for m in log]).tolist()
            room = max_seq_len - len(prompt)
            if room <= 0:
                truncated[i] = True
                return
            sp = dict(sampling)
            sp["max_new_tokens"] = min(int(sp.get("max_new_tokens", 256)), room)
            rec = frontend.submit(prompt, sp)
            toks = torch.tensor(rec.out_tokens, dtype=torch.long)
            text = tokenizer.decode(rec.out_tokens, skip_special_tokens=True) if tokenizer is not None else ""
            log.append({"role": "assistant", "content": text, "token_ids": toks,
                        "generation_logprobs": torch.tensor(rec.out_logprobs, dtype=torch.float32)})
            gen_tokens[i] += toks.numel()
            turns[i] += 1
            truncated[i] = bool(rec.truncated)
            r = env.step([log], [meta])
            rew = r.rewards[0]
            total_reward[i] += float(rew.sum() if rew.dim() else rew)
            meta = r.metadata[0]
            batch["extra_env_info"][i] = meta
            if r.answers is not None:
                answers[i] = r.answers[0]
            if bool(r.terminateds[0]) or turn + 1 >= max_rollout_turns:
                return
            ob = r.observations[0]
            ids = tokenizer(ob["content"], add_special_tokens=False, return_tensors="pt")["input_ids"][0] if tokenizer is not None else torch.empty(0, dtype=torch.long)
            if len(prompt) + toks.numel() + ids.numel() >= max_seq_len:
                truncated[i] = True
                return
            log.append({"role": ob.get("role", "environment"), "content": ob["content"], "token_ids": ids})

    with cf.ThreadPoolExecutor(max_workers=max(1, min(max_concurrency, n))) as pool:
        for f in [pool.submit(one, i) for i in range(n)]:
            f.result()   # re-raises a sample's failure
    batch["total_reward"], batch["truncated"], batch["answers"], batch["generation_lengths"] = total_reward, truncated, answers, gen_tokens
    batch["length"] = torch.tensor([sum(int(m["token_ids"].numel()) for m in log) for log in batch["message_log"]], dtype=torch.long)
    metrics = {"total_turns": int(turns.sum()), "avg_turns_per_sample": float(turns.float().mean()) if n else 0.0,
               "max_turns_per_sample": int(turns.max()) if n else 0, "truncation_rate": float(truncated.float().mean()) if n else 0.0,
               "total_generated_tokens": int(gen_tokens.sum()), "mean_total_reward": float(total_reward.mean()) if n else 0.0}
    return batch, metrics
