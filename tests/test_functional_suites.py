"""The functional and suite tiers stay consistent with the tree: every functional script is driven by the L1 driver, every recipe
is listed in a suite list and every listed recipe exists; the metric checker evaluates what the scripts ask of it; one
functional script runs end to end."""

import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "tests"))


def test_every_functional_script_is_driven():
    d = os.path.join(ROOT, "tests", "functional")
    scripts = sorted(f for f in os.listdir(d) if f.endswith(".sh") and f not in ("common.sh", "L1_Functional_Tests.sh"))
    driver = open(os.path.join(d, "L1_Functional_Tests.sh")).read()
    assert scripts and all(s in driver for s in scripts), [s for s in scripts if s not in driver]
    for s in scripts:
        body = open(os.path.join(d, s)).read()
        assert "run_and_check" in body and " -- " in body.replace("\\\n", " "), s      # a run and at least one assertion


def test_every_recipe_is_listed_in_a_suite():
    base = os.path.join(ROOT, "examples", "configs", "recipes")
    recipes = sorted(os.path.relpath(os.path.join(d, f), base) for d, _, fs in os.walk(base) for f in fs if f.endswith(".yaml"))
    listed = []
    for name in ("nightly.txt", "performance.txt"):
        with open(os.path.join(ROOT, "tests", "test_suites", name)) as f:
            listed += [l.strip() for l in f if l.strip() and not l.startswith("#")]
    assert sorted(listed) == recipes, (sorted(set(recipes) - set(listed)), sorted(set(listed) - set(recipes)))
    assert len(set(listed)) == len(listed)


def test_check_metrics_expressions(tmp_path):
    import check_metrics
    import json_dump_metrics

    log = tmp_path / "logs"
    log.mkdir()
    with open(log / "metrics.jsonl", "w") as f:
        for step, (loss, err) in enumerate([(2.0, 1.01), (1.5, 1.02), (1.0, 1.03)], start=1):
            f.write(json.dumps({"step": step, "train/loss": loss, "train/token_mult_prob_error": err}) + "\n")
            f.write(json.dumps({"step": step, "timing/train/total_step_time": 0.5 * step}) + "\n")
    assert json_dump_metrics.main([str(log), "--output_path", str(tmp_path / "m.json")]) == 0
    data = json.load(open(tmp_path / "m.json"))
    assert data["train/loss"] == {"1": 2.0, "2": 1.5, "3": 1.0}
    ok = ['max(data["train/token_mult_prob_error"]) < 1.05', 'mean(data["train/loss"], 2) == 1.25', 'last(data["train/loss"]) < first(data["train/loss"])',
          'len(data["train/loss"]) == 3', 'ratio_above(data["train/loss"], 1.2) > 0.6', 'mean(data["timing/train/total_step_time"], 2, 3) == 1.25']
    assert check_metrics.main([str(tmp_path / "m.json"), *ok]) == 0
    assert check_metrics.main([str(tmp_path / "m.json"), 'max(data["train/loss"]) < 1', 'min(data["no/such/metric"]) > 0', ok[0]]) == 2
    with pytest.raises(Exception):
        check_metrics.evaluate(data, '__import__("os").system("true")')        # expressions cannot reach beyond the helpers


def test_a_functional_script_runs(tmp_path):
    env = dict(os.environ, RLB_FUNCTIONAL_OUT=str(tmp_path), OMP_NUM_THREADS="4")
    r = subprocess.run(["bash", os.path.join(ROOT, "tests", "functional", "grpo_hybrid.sh")], capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0 and "OK: grpo_hybrid" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
    assert os.path.exists(tmp_path / "grpo_hybrid" / "metrics.json")
