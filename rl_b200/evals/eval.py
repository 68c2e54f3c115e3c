"""Evaluation: pass@k and cons@k over ``num_tests_per_prompt`` samples per prompt (nemo_rl/evals/eval.py:178,206).

``pass@k`` uses the unbiased estimator 1 - C(n-c, k)/C(n, k) over n samples with c correct; ``cons@k`` scores the
majority answer among k samples (expected value over k-subsets, estimated from all n when k == n).
"""

from __future__ import annotations

import json
import math
from collections import Counter
from typing import Optional

import torch

from rl_b200.algorithms.grpo import _all_reduce_scalars, _is_main, _world
from rl_b200.experience.rollouts import run_multi_turn_rollout


def eval_pass_k(rewards: torch.Tensor, num_tests_per_prompt: int, k: int) -> float:
    """Sum over prompts of the unbiased pass@k estimate. ``rewards``: [num_prompts * n], grouped by prompt."""
    n = num_tests_per_prompt
    assert 1 <= k <= n
    c = (rewards.view(-1, n) >= 1.0).sum(dim=1).tolist()
    return float(sum(1.0 - (math.comb(n - ci, k) / math.comb(n, k) if n - ci >= k else 0.0) for ci in c))


def eval_cons_k(rewards: torch.Tensor, num_tests_per_prompt: int, k: int, answers: list) -> float:
    """Sum over prompts of the majority-vote score using the first k samples of every prompt."""
    n = num_tests_per_prompt
    assert 1 <= k <= n
    r = rewards.view(-1, n)
    total = 0.0
    for i in range(r.shape[0]):
        ans = answers[i * n : i * n + k]
        valid = [a for a in ans if a is not None]
        if not valid:
            continue
        top = Counter(valid).most_common(1)[0][0]
        j = ans.index(top)
        total += float(r[i, j] >= 1.0)
    return total


def run_env_eval(generation, loader, tokenizer, task_to_env, cfg: dict) -> dict:
    """Generates ``num_tests_per_prompt`` samples per validation prompt, scores them with the environment and reports
    ``score`` under ``metric`` (``pass@k`` or ``cons@k``). Returns a dict; rank 0 may dump per-sample records."""
    e = dict(metric="pass@k", num_tests_per_prompt=1, k_value=1, seed=42, save_path=None)
    e.update(cfg.get("eval") or {})
    rank, world = _world()
    pad = tokenizer.pad_token_id if tokenizer.pad_token_id is not None else 0
    n = int(e["num_tests_per_prompt"])
    score, count, records = 0.0, 0, []
    generation.prepare_for_generation()
    for batch in loader:
        rep = batch.repeat_interleave(n)
        rep["message_log"] = [[dict(m) for m in log] for log in rep["message_log"]]
        rep["rng_ids"] = rep["idx"] * n + torch.arange(n).repeat(batch.size)
        rep, _ = run_multi_turn_rollout(generation, rep, tokenizer, task_to_env, cfg["policy"]["max_total_sequence_length"],
                                        max_rollout_turns=1, greedy=(n == 1 and (cfg["policy"].get("generation") or {}).get("temperature", 1.0) == 0),
                                        pad_token_id=pad)
        rewards = rep["total_reward"].float()
        if e["metric"] == "pass@k":
            score += eval_pass_k(rewards, n, int(e["k_value"]))
        elif e["metric"] == "cons@k":
            answers = list(rep.get("answers") or [None] * rep.size)
            score += eval_cons_k(rewards, n, int(e["k_value"]), answers)
        else:
            raise ValueError(f"unknown eval metric {e['metric']}")
        count += batch.size
        if e.get("save_path") and _is_main():
            for i, log in enumerate(rep["message_log"]):
                records.append({"idx": int(rep["idx"][i]), "reward": float(rewards[i]),
                                "response": "".join(str(m["content"]) for m in log if m["role"] == "assistant")})
    generation.finish_generation()
    tot = _all_reduce_scalars({"s": score, "n": float(count)})
    out = {"metric": f"{e['metric'].split('@')[0]}@{e['k_value']}", "score": tot["s"] / max(1.0, tot["n"]), "num_prompts": int(tot["n"]),
           "num_tests_per_prompt": n}
    if e.get("save_path") and _is_main():
        with open(e["save_path"], "w") as f:
            json.dump({"summary": out, "samples": records}, f, indent=1)
    return out
