"""On-policy distillation inside GRPO: teachers score the student's own rollouts and the per-token advantage is
``teacher logprob - student logprob`` (:class:`rl_b200.algorithms.advantage_estimator.OPDAdvantageEstimator`).

This module holds what surrounds the estimator: the ``on_policy_distillation`` config block, the routing of every sample
to a teacher by the agent (task) that produced it, de-duplication of aliases that share a checkpoint, the frozen
inference-only teacher workers and the routing diagnostics. It follows nemo_rl/algorithms/opd.py:40-214 (config and
routing) and nemo_rl/models/policy/teacher_worker_group.py:43-308 (inference-only teacher groups); the teachers here are
frozen :class:`rl_b200.policy.worker.PolicyWorker` instances on the training ranks' own GPUs (no optimizer, no reference
copy), one per distinct checkpoint.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional, Sequence

import torch

from rl_b200.distributed.batched_data_dict import BatchedDataDict

OPD_DEFAULTS = dict(teacher_model_by_agent_name={}, default_teacher_alias=None, deduplicate_shared_teacher_checkpoints=True,
                    non_colocated_teachers=None)
TEACHER_RESOURCE_DEFAULTS = dict(tensor_model_parallel_size=1, pipeline_model_parallel_size=1, context_parallel_size=1,
                                 expert_model_parallel_size=1, num_nodes=1, gpus_per_node=8, precision="bfloat16", micro_batch_size=1)


def opd_cfg(master_config: dict) -> dict:
    out = dict(OPD_DEFAULTS)
    out.update(master_config.get("on_policy_distillation") or {})
    return out


def is_opd_enabled(master_config: dict) -> bool:
    name = ((master_config.get("grpo") or {}).get("adv_estimator") or {}).get("name")
    return name == "opd"


def is_non_colocated_teachers_enabled(master_config: dict) -> bool:
    return bool((opd_cfg(master_config).get("non_colocated_teachers") or {}).get("enabled", False))


@dataclass
class TeacherConfig:
    """One teacher after defaults, per-alias overrides and de-duplication."""

    alias: str
    model_name: str
    tensor_model_parallel_size: int = 1
    pipeline_model_parallel_size: int = 1
    context_parallel_size: int = 1
    expert_model_parallel_size: int = 1
    num_nodes: int = 1
    gpus_per_node: int = 8
    precision: str = "bfloat16"
    micro_batch_size: int = 1
    overrides: dict = field(default_factory=dict)


def create_teacher_configs(cfg: dict) -> list[TeacherConfig]:
    """``teacher_model_by_agent_name`` (alias -> checkpoint) -> one config per teacher to load. With
    ``deduplicate_shared_teacher_checkpoints`` aliases that name the same checkpoint share the first alias's teacher."""
    by_alias = dict(cfg.get("teacher_model_by_agent_name") or {})
    nc = dict(cfg.get("non_colocated_teachers") or {})
    default = dict(TEACHER_RESOURCE_DEFAULTS)
    default.update(nc.get("default_teacher_cfg") or {})
    per_alias = dict(nc.get("teacher_overrides") or {})
    dedup = bool(cfg.get("deduplicate_shared_teacher_checkpoints", True))
    out, seen = [], set()
    for alias, model in by_alias.items():
        if dedup and model in seen:
            continue
        seen.add(model)
        merged = dict(default)
        merged.update(per_alias.get(alias) or {})
        known = {k: merged.pop(k) for k in list(merged) if k in TEACHER_RESOURCE_DEFAULTS}
        extra = dict(merged.pop("megatron_cfg_overrides", {}) or {})
        merged.update(extra)             # unknown keys are worker-config overrides
        out.append(TeacherConfig(alias=alias, model_name=model, overrides=merged, **known))
    return out


def alias_to_group_alias(cfg: dict) -> dict[str, str]:
    """alias -> alias of the teacher that serves it (differs only for de-duplicated aliases)."""
    by_alias = dict(cfg.get("teacher_model_by_agent_name") or {})
    if not cfg.get("deduplicate_shared_teacher_checkpoints", True):
        return {a: a for a in by_alias}
    first: dict[str, str] = {}
    out = {}
    for a, m in by_alias.items():
        first.setdefault(m, a)
        out[a] = first[m]
    return out


def resolve_teacher_aliases(agent_names: Sequence[Optional[str]], teacher_model_by_agent_name: dict[str, str],
                            default_teacher_alias: Optional[str] = None) -> list[str]:
    """The teacher alias of every sample. Agents without a mapping fall back to ``default_teacher_alias`` or fail."""
    out = []
    for name in agent_names:
        if name in teacher_model_by_agent_name:
            out.append(name)
        elif default_teacher_alias:
            if default_teacher_alias not in teacher_model_by_agent_name:
                raise KeyError(f"default_teacher_alias '{default_teacher_alias}' has no teacher model")
            out.append(default_teacher_alias)
        else:
            raise KeyError(f"no teacher model for agent '{name}' and no default_teacher_alias; known: {sorted(teacher_model_by_agent_name)}")
    return out


def teacher_routing_metrics(aliases: Sequence[str], teacher_model_by_agent_name: dict[str, str]) -> dict[str, float]:
    models = set()
    for a in aliases:
        if a not in teacher_model_by_agent_name:
            raise KeyError(f"alias '{a}' not found in teacher_model_by_agent_name")
        models.add(teacher_model_by_agent_name[a])
    ua = len(set(aliases))
    return {"on_policy_distillation/teacher_alias_unique": float(ua), "on_policy_distillation/teacher_model_unique": float(len(models)),
            "on_policy_distillation/teacher_alias_to_model_compression": float(ua) / max(1, len(models))}


class TeacherGroup:
    """A frozen, inference-only teacher: loads its checkpoint once, never builds an optimizer or a reference copy, and only
    answers ``get_logprobs``."""

    def __init__(self, tcfg: TeacherConfig, policy_config: dict, tokenizer=None, model_cfg=None, worker=None):
        from rl_b200.policy.worker import PolicyWorker

        self.alias, self.model_name, self.cfg = tcfg.alias, tcfg.model_name, tcfg
        if worker is None:
            cfg = {k: v for k, v in policy_config.items() if k not in ("optimizer", "scheduler", "generation", "lora_cfg")}
            cfg.update(model_name=tcfg.model_name, precision=tcfg.precision, logprob_batch_size=tcfg.micro_batch_size)
            cfg.update(tcfg.overrides)
            worker = PolicyWorker(cfg, model_cfg=model_cfg, tokenizer=tokenizer, init_optimizer=False, init_reference_model=False,
                                  weights_path=tcfg.model_name if model_cfg is None else None)
        self.worker = worker
        for p in self.worker.model.parameters():
            p.requires_grad_(False)

    def get_logprobs(self, data: BatchedDataDict, micro_batch_size: Optional[int] = None) -> BatchedDataDict:
        return BatchedDataDict(reference_logprobs=self.worker.get_logprobs(data, micro_batch_size)["logprobs"])

    def shutdown(self) -> bool:
        return self.worker.shutdown()


def create_teacher_groups(master_config: dict, tokenizer=None, model_cfg=None) -> tuple[dict[str, TeacherGroup], dict[str, str]]:
    cfg = opd_cfg(master_config)
    if is_non_colocated_teachers_enabled(master_config) and not (torch.distributed.is_available() and torch.distributed.is_initialized()
                                                                 and torch.distributed.get_world_size() > 1):
        # teachers on GPUs of their own, driven from this (single controller) process through worker groups
        from dataclasses import asdict

        from rl_b200.policy.lm_policy import create_teacher_worker_groups

        return create_teacher_worker_groups(master_config, asdict(model_cfg) if model_cfg is not None else None,
                                            (master_config.get("policy") or {}).get("tokenizer"),
                                            (master_config.get("cluster") or {}).get("backend"))
    groups = {t.alias: TeacherGroup(t, master_config["policy"], tokenizer, model_cfg) for t in create_teacher_configs(cfg)}
    return groups, alias_to_group_alias(cfg)


def compute_teacher_logprobs(train_data: BatchedDataDict, agent_names: Sequence[Optional[str]], groups: dict[str, TeacherGroup],
                             alias_map: dict[str, str], cfg: dict) -> tuple[torch.Tensor, dict[str, float]]:
    """Teacher log-probabilities [B, S] of the sampled tokens: every sample is scored by the teacher of its agent. Samples
    are grouped by teacher so that each teacher runs once over its own rows."""
    by_alias = dict(cfg.get("teacher_model_by_agent_name") or {})
    aliases = resolve_teacher_aliases(agent_names, by_alias, cfg.get("default_teacher_alias"))
    out = torch.zeros(train_data["input_ids"].shape, dtype=torch.float32)
    rows_of: dict[str, list[int]] = {}
    for i, a in enumerate(aliases):
        rows_of.setdefault(alias_map.get(a, a), []).append(i)
    for g_alias, rows in rows_of.items():
        sub = train_data.select_indices(rows) if hasattr(train_data, "select_indices") else BatchedDataDict(
            {k: (v[rows] if isinstance(v, torch.Tensor) else [v[i] for i in rows]) for k, v in train_data.items()})
        lp = groups[g_alias].get_logprobs(sub)["reference_logprobs"]
        out[torch.tensor(rows), : lp.shape[1]] = lp.float().cpu()
    return out, teacher_routing_metrics(aliases, by_alias)
