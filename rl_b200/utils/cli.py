"""Shared bootstrap of the example entrypoints: ``--config`` + Hydra-style overrides -> resolved config, process group,
tokenizer (nemo_rl's examples do the same with OmegaConf + ``init_ray``: examples/run_grpo.py:71-254)."""

from __future__ import annotations

import os
import pprint
from typing import Optional

from rl_b200.distributed.launch import init_distributed
from rl_b200.utils.config import load_config, parse_args_and_overrides


def apply_env_vars(cfg: dict) -> dict:
    """Recipe ``env_vars`` override the shell; the policy's own blocks (``policy.env_vars``, ``policy.dtensor_cfg.env_vars``,
    ``policy.megatron_cfg.env_vars``, ``policy.generation.*_cfg.env_vars``) override the recipe's top level, in that order
    (the reference's precedence: docs/design-docs/env-vars.md:5-31). Returns what was set."""
    pol = cfg.get("policy") or {}
    gen = pol.get("generation") or {}
    layers = [cfg.get("env_vars"), pol.get("env_vars"), (pol.get("dtensor_cfg") or {}).get("env_vars"),
              (pol.get("megatron_cfg") or {}).get("env_vars"), (gen.get("native_cfg") or {}).get("env_vars"),
              (gen.get("vllm_cfg") or {}).get("env_vars")]
    applied = {}
    for layer in layers:
        for k, v in (layer or {}).items():
            os.environ[str(k)] = str(v)
            applied[str(k)] = str(v)
    return applied


def bootstrap(default_config: str, argv: Optional[list[str]] = None, backend: Optional[str] = None):
    """Returns (cfg, rank, world, device, tokenizer)."""
    path, overrides = parse_args_and_overrides(argv)
    cfg = load_config(path or default_config, overrides)
    apply_env_vars(cfg)
    validate_recipe(cfg, quiet=int(os.environ.get("RANK", "0")) != 0)
    from rl_b200.distributed import roles

    layout = roles.init_roles(cfg, backend or (cfg.get("cluster") or {}).get("backend"))
    roles.set_current_layout(layout)
    rank, world, device = layout.role_rank, layout.role_world, layout.device   # coordinates inside this rank's own set
    if rank == 0:
        print(f"Loaded configuration from {path or default_config}")
        pprint.pprint(cfg, width=140, compact=True)
    from rl_b200.algorithms.utils import get_tokenizer

    tcfg = (cfg.get("policy") or {}).get("tokenizer") or {"name": "byte"}
    tokenizer = get_tokenizer(tcfg)
    return cfg, rank, world, device, tokenizer


def model_cfg_for_tokenizer(cfg: dict, tokenizer):
    """When the config asks for a preset architecture with a byte tokenizer, shrink the vocabulary to the tokenizer's."""
    from rl_b200.models.config import PRESETS, preset

    pcfg = cfg["policy"]
    name = pcfg.get("model_name")
    if name in PRESETS:
        over = dict(pcfg.get("hf_config_overrides") or {})
        if getattr(tokenizer, "name_or_path", None) in ("byte", "pair"):
            over.setdefault("vocab_size", len(tokenizer))
        return preset(name, **over)
    return None


def infer_algorithm(cfg: dict) -> str:
    """Which algorithm's schema a recipe follows, from the sections it contains."""
    for name in ("ppo", "distillation", "dpo", "rm", "sft", "grpo", "eval"):
        if name in cfg:
            return name
    return "grpo"


def validate_recipe(cfg: dict, quiet: bool = False):
    """Typed validation of a loaded recipe (rl_b200/config/schema.py): wrong types and missing required keys stop the
    run, keys that nothing reads are listed once with the closest known key."""
    from rl_b200.config.schema import validate_master_config

    return validate_master_config(cfg, infer_algorithm(cfg), strict=os.environ.get("RLB_STRICT_CONFIG", "0") == "1", quiet=quiet)
