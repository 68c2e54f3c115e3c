"""YAML loader: inheritance, _override_, interpolation / resolvers, Hydra-style overrides."""

import pytest
import yaml

from rl_b200.utils.config import ConfigError, apply_overrides, deep_merge, load_config, resolve


def _write(p, d):
    p.write_text(yaml.safe_dump(d))
    return p


def test_inheritance_and_override_marker(tmp_path):
    _write(tmp_path / "base.yaml", {"policy": {"lr": 1.0, "opt": {"name": "adam", "kwargs": {"a": 1, "b": 2}}}, "x": 1})
    _write(tmp_path / "mid.yaml", {"defaults": "base.yaml", "policy": {"lr": 2.0}})
    _write(tmp_path / "child.yaml", {"defaults": ["mid.yaml"], "policy": {"opt": {"_override_": True, "name": "sgd"}}, "y": "${mul:${x},3}"})
    cfg = load_config(tmp_path / "child.yaml")
    assert cfg["policy"]["lr"] == 2.0
    assert cfg["policy"]["opt"] == {"name": "sgd"}  # replaced, not merged
    assert cfg["y"] == 3 and cfg["x"] == 1


def test_interpolation_and_resolvers():
    cfg = resolve({"a": {"b": 4}, "c": "${a.b}", "d": "${add:${a.b},1}", "e": "p_${a.b}_s", "f": "${div:${a.b},8}", "g": "${max:1,${a.b}}"})
    assert cfg["c"] == 4 and cfg["d"] == 5 and cfg["e"] == "p_4_s" and cfg["f"] == 0.5 and cfg["g"] == 4
    with pytest.raises(ConfigError):
        resolve({"a": "${a}"})
    with pytest.raises(ConfigError):
        resolve({"a": "${nope.key}"})


def test_overrides():
    cfg = {"a": {"b": 1, "l": [1, 2]}, "k": None}
    out = apply_overrides(cfg, ["a.b=2", "+a.c=[1,2]", "++a.d.e=true", "~k", "a.l.0=9"])
    assert out == {"a": {"b": 2, "l": [9, 2], "c": [1, 2], "d": {"e": True}}}
    assert cfg["a"]["b"] == 1  # input untouched
    with pytest.raises(ConfigError):
        apply_overrides(cfg, ["a.zzz=1"])
    with pytest.raises(ConfigError):
        apply_overrides(cfg, ["+a.b=1"])


def test_deep_merge_lists_replace():
    assert deep_merge({"a": [1, 2], "b": {"c": 1}}, {"a": [3], "b": {"d": 2}}) == {"a": [3], "b": {"c": 1, "d": 2}}


def test_circular_defaults(tmp_path):
    _write(tmp_path / "a.yaml", {"defaults": "b.yaml"})
    _write(tmp_path / "b.yaml", {"defaults": "a.yaml"})
    with pytest.raises(ConfigError):
        load_config(tmp_path / "a.yaml")


def test_env_vars_precedence(monkeypatch):
    import os

    from rl_b200.utils.cli import apply_env_vars

    monkeypatch.setenv("RLB_TEST_A", "shell")
    monkeypatch.setenv("RLB_TEST_B", "shell")
    monkeypatch.setenv("RLB_TEST_C", "shell")
    cfg = dict(env_vars=dict(RLB_TEST_A="recipe", RLB_TEST_B="recipe"),
               policy=dict(dtensor_cfg=dict(env_vars=dict(RLB_TEST_B="worker")), generation=dict(vllm_cfg=dict(env_vars=dict(RLB_TEST_D=1)))))
    applied = apply_env_vars(cfg)
    assert os.environ["RLB_TEST_A"] == "recipe" and os.environ["RLB_TEST_B"] == "worker" and os.environ["RLB_TEST_C"] == "shell"
    assert os.environ["RLB_TEST_D"] == "1" and applied["RLB_TEST_B"] == "worker"
    for k in ("RLB_TEST_D",):
        monkeypatch.delenv(k, raising=False)
