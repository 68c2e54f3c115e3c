"""Step-time and throughput table from a run's ``metrics.jsonl`` (the logger's JSON-lines backend): averages of the step
phases and tokens/s/GPU over a window of steps, in the shape of the reference's performance summary
(docs/about/performance-summary.md; tools/wandb_to_perf_numbers.py reads the same keys from W&B).

    python -m rl_b200.tools.perf_numbers logs/exp_001 --at-step 6 --average-steps 5 [--json]
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Iterable

KEYS = (
    "train/total_num_tokens",
    "timing/train/total_step_time",
    "timing/train/generation",
    "timing/train/policy_training",
    "timing/train/policy_and_reference_logprobs",
    "timing/train/prepare_for_generation/total",
    "timing/train/reward_calculation",
    "timing/train/checkpointing",
    "performance/tokens_per_sec_per_gpu",
    "performance/generation_tokens_per_sec_per_gpu",
    "performance/policy_training_tokens_per_sec_per_gpu",
    "performance/policy_and_reference_logprobs_tokens_per_sec_per_gpu",
    "performance/train_flops_per_gpu",
    "performance/train_fp_utilization",
    "train/token_mult_prob_error",
)


def read_metrics(path: str) -> dict[int, dict[str, float]]:
    """step -> merged scalars (the logger writes one line per ``log_metrics`` call: ``{"step": n, ...}``)."""
    if os.path.isdir(path):
        path = os.path.join(path, "metrics.jsonl")
    out: dict[int, dict[str, float]] = {}
    with open(path) as f:
        for line in f:
            line = line.strip()
            if not line:
                continue
            rec = json.loads(line)
            step = int(rec.get("step", rec.get("_step", -1)))
            out.setdefault(step, {}).update({k: v for k, v in rec.items() if isinstance(v, (int, float)) and k not in ("step", "_step")})
    return out


def window(at_step: int, average_steps: int) -> range:
    lo = at_step - average_steps // 2
    hi = at_step + average_steps // 2 - 1 + (average_steps % 2)
    return range(lo, hi + 1)


def summarize(metrics: dict[int, dict[str, float]], at_step: int = 6, average_steps: int = 5, keys: Iterable[str] = KEYS) -> dict:
    steps = [s for s in window(at_step, average_steps) if s in metrics]
    if not steps:
        raise ValueError(f"no logged step in {list(window(at_step, average_steps))} (logged: {sorted(metrics)[:5]}...{sorted(metrics)[-3:]})")
    table = {}
    for k in keys:
        vals = [metrics[s][k] for s in steps if k in metrics[s]]
        if vals:
            table[k] = sum(vals) / len(vals)
    return dict(steps=steps, averages=table)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("log_dir")
    ap.add_argument("--at-step", type=int, default=6)
    ap.add_argument("--average-steps", type=int, default=5)
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)
    res = summarize(read_metrics(a.log_dir), a.at_step, a.average_steps)
    if a.json:
        print(json.dumps(res))
    else:
        print(f"steps {res['steps'][0]}..{res['steps'][-1]} ({len(res['steps'])} logged)")
        for k, v in res["averages"].items():
            print(f"{k:70s} {v:14.4f}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
