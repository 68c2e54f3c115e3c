"""Typed recipe validation: wrong types and missing keys are errors, a misspelt key is reported with the closest known
key, every recipe shipped with the framework validates, and so do recipes written for the reference."""

import glob
import os

import pytest

from rl_b200.config.schema import ConfigError, POLICY, validate, validate_master_config
from rl_b200.utils.cli import infer_algorithm
from rl_b200.utils.config import load_config

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _base():
    return dict(policy=dict(train_global_batch_size=8, train_micro_batch_size=2, max_total_sequence_length=128, precision="bfloat16",
                            generation=dict(max_new_tokens=16, temperature=1.0, colocated=dict(enabled=True))),
                loss_fn=dict(ratio_clip_min=0.2, ratio_clip_max=0.2, reference_policy_kl_penalty=0.01),
                grpo=dict(num_prompts_per_step=4, num_generations_per_prompt=2), checkpointing=dict(enabled=False),
                logger=dict(log_dir="logs"), cluster=dict(gpus_per_node=1, num_nodes=1))


def test_valid_recipe_passes_and_reports_nothing():
    rep = validate_master_config(_base(), "grpo", quiet=True)
    assert rep.ok() and not rep.unknown


def test_misspelt_key_is_listed_with_a_suggestion(capsys):
    cfg = _base()
    cfg["policy"]["train_micro_batchsize"] = 4           # typo of train_micro_batch_size
    cfg["grpo"]["num_generation_per_prompt"] = 8         # typo
    rep = validate_master_config(cfg, "grpo")
    found = dict(rep.unknown)
    assert found["policy.train_micro_batchsize"] == "train_micro_batch_size"
    assert found["grpo.num_generation_per_prompt"] == "num_generations_per_prompt"
    out = capsys.readouterr().out
    assert "did you mean 'train_micro_batch_size'" in out
    # listed once per process: a second validation of the same recipe prints nothing
    validate_master_config(cfg, "grpo")
    assert "did you mean" not in capsys.readouterr().out
    with pytest.raises(ConfigError, match="num_generation_per_prompt"):
        validate_master_config(cfg, "grpo", strict=True, quiet=True)


def test_type_errors_missing_keys_and_choices_stop_the_run():
    cfg = _base()
    cfg["policy"]["train_global_batch_size"] = "eight"
    cfg["policy"]["generation"]["temperature"] = [1.0]
    cfg["loss_fn"]["reference_policy_kl_type"] = "k9"
    cfg["grpo"]["normalize_rewards"] = 1                 # an int is not a bool
    del cfg["policy"]["max_total_sequence_length"]
    with pytest.raises(ConfigError) as e:
        validate_master_config(cfg, "grpo", quiet=True)
    msg = str(e.value)
    for needle in ("policy.train_global_batch_size: expected int", "policy.generation.temperature", "'k9' is not one of",
                   "grpo.normalize_rewards: expected bool", "policy.max_total_sequence_length: required key is missing"):
        assert needle in msg, needle


def test_numeric_strings_and_ints_for_floats_are_accepted():
    rep = validate("policy", dict(train_global_batch_size=8, train_micro_batch_size=1, max_total_sequence_length=64, max_grad_norm=1,
                                  megatron_cfg=dict(enabled=False, moe_router_bias_update_rate="1e-3")), POLICY)
    assert rep.ok()


def test_every_shipped_recipe_validates():
    paths = sorted(glob.glob(os.path.join(ROOT, "examples", "configs", "**", "*.yaml"), recursive=True))
    assert len(paths) >= 20
    for p in paths:
        cfg = load_config(p, [])
        validate_master_config(cfg, infer_algorithm(cfg), quiet=True)


_REF_CONFIGS = os.environ.get("RLB_REFERENCE_CONFIGS", "")   # a directory of recipes written for the reference implementation


@pytest.mark.skipif(not os.path.isdir(_REF_CONFIGS), reason="set RLB_REFERENCE_CONFIGS to a directory of reference recipes")
def test_reference_recipes_validate_without_errors():
    paths = sorted(glob.glob(os.path.join(_REF_CONFIGS, "*.yaml")))
    for p in paths:
        cfg = load_config(p, [])
        validate_master_config(cfg, infer_algorithm(cfg), quiet=True)
