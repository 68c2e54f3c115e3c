"""Dumps a run's ``metrics.jsonl`` as ``{metric: {step: value}}`` JSON, the input of ``check_metrics.py`` (the role of the
reference's tests/json_dump_tb_logs.py for the TensorBoard backend).

    python tests/json_dump_metrics.py logs/exp --output_path metrics.json
"""

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def dump(log_dir: str) -> dict:
    from rl_b200.tools.perf_numbers import read_metrics

    path = log_dir
    if os.path.isdir(log_dir) and not os.path.exists(os.path.join(log_dir, "metrics.jsonl")):
        hits = sorted(os.path.join(d, f) for d, _, fs in os.walk(log_dir) for f in fs if f == "metrics.jsonl")
        if not hits:
            raise FileNotFoundError(f"no metrics.jsonl under {log_dir}")
        path = hits[-1]
    out: dict = {}
    for step, vals in sorted(read_metrics(path).items()):
        for k, v in vals.items():
            out.setdefault(k, {})[str(step)] = v
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("log_dir")
    ap.add_argument("--output_path", required=True)
    a = ap.parse_args(argv)
    data = dump(a.log_dir)
    with open(a.output_path, "w") as f:
        json.dump(data, f, indent=1)
    print(f"wrote {len(data)} metrics to {a.output_path}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
