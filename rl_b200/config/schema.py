"""Typed configuration schema: every section of a recipe is checked against a table of fields before a run starts.

A schema is a mapping ``name -> Field``. ``validate(section, cfg, schema)`` checks the type of every known key, fills
nothing in (defaults stay where the consumers define them), and collects two kinds of findings:

  * errors: a known key with a value of the wrong type, a missing required key, a value outside its choices;
  * unknown keys: allowed (recipes written for the reference carry keys for back ends that do not exist here), but
    listed ONCE at start-up together with the closest known key, so that a misspelt key never passes silently.

``validate_master_config(cfg, algorithm)`` walks the whole recipe (policy, generation, loss, algorithm section,
checkpointing, logger, cluster, data) and raises ``ConfigError`` on errors. The entry points call it right after the
YAML is loaded. The tables below follow the reference's ``PolicyConfig`` / ``GRPOConfig`` / ``MasterConfig``
(nemo_rl/models/policy/__init__.py:562-608, nemo_rl/algorithms/grpo.py:241-368) key for key; keys of back ends that are
not built here (Megatron, vLLM, SGLang internals) are accepted as opaque sub-sections.
"""

from __future__ import annotations

import difflib
from dataclasses import dataclass, field
from typing import Any, Optional, Sequence

_NUM = (int, float)


class ConfigError(ValueError):
    """A recipe failed validation; the message lists every finding."""


@dataclass(frozen=True)
class Field:
    types: tuple = (object,)          # accepted python types (bool is never accepted where only int / float is named)
    required: bool = False
    nullable: bool = True
    choices: Optional[tuple] = None
    sub: Optional[dict] = None        # schema of a nested section (dict value)
    item: Optional[dict] = None       # schema of every element of a list of sections
    doc: str = ""


def F(*types, required=False, nullable=True, choices=None, sub=None, item=None, doc="") -> Field:
    return Field(tuple(types) or (object,), required, nullable, tuple(choices) if choices else None, sub, item, doc)


@dataclass
class Report:
    errors: list = field(default_factory=list)
    unknown: list = field(default_factory=list)   # (path, suggestion or None)

    def ok(self) -> bool:
        return not self.errors

    def render(self) -> str:
        lines = [f"error: {e}" for e in self.errors]
        for path, hint in self.unknown:
            lines.append(f"unknown key: {path}" + (f" (did you mean '{hint}'?)" if hint else ""))
        return "\n".join(lines)


def _type_ok(v: Any, types: tuple) -> bool:
    if object in types:
        return True
    if isinstance(v, bool):
        return bool in types
    if isinstance(v, int) and float in types:
        return True
    if isinstance(v, str) and float in types and str not in types:
        try:   # YAML 1.1 reads "1e-3" (no dot) as a string; the consumers convert with float()
            float(v)
            return True
        except ValueError:
            return False
    return isinstance(v, tuple(t for t in types if t is not bool) or (bool,))


def _names(types: tuple) -> str:
    return " | ".join(getattr(t, "__name__", str(t)) for t in types)


def validate(path: str, cfg: Any, schema: dict, report: Optional[Report] = None) -> Report:
    """Checks ``cfg`` (a mapping) against ``schema``; findings go to ``report`` with ``path`` as prefix."""
    rep = report if report is not None else Report()
    if cfg is None:
        return rep
    if not isinstance(cfg, dict):
        rep.errors.append(f"{path}: expected a mapping, got {type(cfg).__name__}")
        return rep
    for name, f in schema.items():
        if name not in cfg:
            if f.required:
                rep.errors.append(f"{path}.{name}: required key is missing")
            continue
        v = cfg[name]
        here = f"{path}.{name}"
        if v is None:
            if not f.nullable:
                rep.errors.append(f"{here}: must not be null")
            continue
        if not _type_ok(v, f.types):
            rep.errors.append(f"{here}: expected {_names(f.types)}, got {type(v).__name__} ({v!r})")
            continue
        if f.choices is not None and v not in f.choices:
            rep.errors.append(f"{here}: {v!r} is not one of {list(f.choices)}")
        if f.sub is not None and isinstance(v, dict):
            validate(here, v, f.sub, rep)
        if f.item is not None and isinstance(v, (list, tuple)):
            for i, x in enumerate(v):
                if isinstance(x, dict):
                    validate(f"{here}[{i}]", x, f.item, rep)
    known = list(schema)
    for k in cfg:
        if k not in schema:
            close = difflib.get_close_matches(str(k), known, n=1, cutoff=0.75)
            rep.unknown.append((f"{path}.{k}", close[0] if close else None))
    return rep


# ------------------------------------------------------------------------------------------------ the tables
OPAQUE = F(dict)   # a sub-section that is passed through (back ends that are not built here)

TOKENIZER = dict(use_fastokens=F(bool), name=F(str), chat_template=F(str), chat_template_kwargs=F(dict), padding_side=F(str, choices=("left", "right")),
                 type=F(str), path=F(str), vocab_size=F(int), words=F(list))

PARALLEL = dict(tensor_parallel_size=F(int, nullable=False), pipeline_parallel_size=F(int), context_parallel_size=F(int),
                expert_parallel_size=F(int), sequence_parallel=F(bool), virtual_pipeline_stages=F(int),
                data_parallel_replicate_size=F(int), data_parallel_sharding=F(str, choices=("optimizer", "full")), hsdp_replicas=F(int))

LORA = dict(enabled=F(bool), dim=F(int), alpha=F(int, float), dropout=F(float, int), target_modules=F(list), exclude_modules=F(list),
            match_all_linear=F(bool), dropout_position=F(str), lora_A_init=F(str), use_triton=F(bool), rank=F(int),
            lora_A_init_method=F(str), lora_B_init_method=F(str), a2a_experimental=F(bool), lora_dtype=F(str))

FP8 = dict(enabled=F(bool), fp8=F(str, choices=("e4m3", "hybrid")), fp8_recipe=F(str, choices=("mxfp8", "blockwise", "tensorwise", "delayed")),
           fp8_param=F(bool), force_clear_fp8_caches=F(bool))

DTENSOR = dict(enabled=F(bool), _v2=F(bool), cpu_offload=F(bool), sequence_parallel=F(bool), activation_checkpointing=F(bool),
               tensor_parallel_size=F(int), context_parallel_size=F(int), expert_parallel_size=F(int), custom_parallel_plan=F(str),
               clear_cache_every_n_steps=F(int), lora_cfg=F(dict, sub=LORA), env_vars=F(dict), automodel_kwargs=F(dict),
               data_parallel_sharding=F(str, choices=("optimizer", "full")), hsdp_replicas=F(int), dp_replicate_size=F(int), defer_fsdp_grad_sync=F(bool),
               moe_parallelizer=F(dict), fp8_cfg=F(dict, sub=FP8))

MEGATRON = dict(enabled=F(bool), tensor_model_parallel_size=F(int), pipeline_model_parallel_size=F(int), context_parallel_size=F(int),
                expert_model_parallel_size=F(int), expert_tensor_parallel_size=F(int), sequence_parallel=F(bool),
                num_layers_in_first_pipeline_stage=F(int), num_layers_in_last_pipeline_stage=F(int),
                virtual_pipeline_model_parallel_size=F(int), activation_checkpointing=F(bool), empty_unused_memory_level=F(int),
                freeze_moe_router=F(bool), moe_router_dtype=F(str), moe_router_load_balancing_type=F(str), moe_router_bias_update_rate=F(float, int),
                moe_permute_fusion=F(bool), moe_per_layer_logging=F(bool), moe_token_dispatcher_type=F(str), moe_shared_expert_overlap=F(bool),
                moe_enable_deepep=F(bool), apply_rope_fusion=F(bool), bias_activation_fusion=F(bool), defer_fp32_logits=F(bool),
                pipeline_dtype=F(str), converter_type=F(str), train_iters=F(int), fp8_cfg=F(dict, sub=FP8), optimizer=OPAQUE, scheduler=OPAQUE,
                distributed_data_parallel_config=OPAQUE, env_vars=F(dict), peft=F(dict, sub=LORA), checkpoint=OPAQUE,
                gradient_accumulation_fusion=F(bool), linear_ce_fusion=F(bool), force_overwrite_initial_ckpt=F(bool),
                use_custom_fsdp=F(bool), layernorm_epsilon=F(float), mtp_loss_scaling_factor=F(float, int), mtp_num_layers=F(int),
                # accepted for the reference's recipes; no component here reads them
                use_fused_weighted_squared_relu=F(bool), fine_grained_activation_offloading=F(bool), offload_modules=F(list),
                use_gloo_process_groups=F(bool), force_reconvert_from_hf=F(bool), cuda_graph_impl=F(str), cuda_graph_modules=F(list),
                cuda_graph_warmup_steps=F(int), recompute_granularity=F(str), recompute_modules=F(list), use_fused_linear_logprobs=F(bool),
                fused_linear_logprobs_chunk_size=F(int), mtp_use_repeated_layer=F(bool), mtp_detach_heads=F(bool), model_overrides=F(dict),
                moe_grouped_gemm=F(bool), moe_router_enable_expert_bias=F(bool))

PACKING = dict(enabled=F(bool), train_mb_tokens=F(int), logprob_mb_tokens=F(int), algorithm=F(str, choices=(
    "concatenative", "first_fit_decreasing", "first_fit_shuffle", "modified_first_fit_decreasing", "modified_ffd", "best_fit_decreasing")),
    microbatch_order=F(str), fuse_loss=F(bool),
    sequence_length_round=F(int))

DYNAMIC_BATCHING = dict(enabled=F(bool), train_mb_tokens=F(int), logprob_mb_tokens=F(int), sequence_length_round=F(int))

OPTIMIZER = dict(name=F(str, required=True), kwargs=F(dict))

SCHEDULER_ITEM = dict(name=F(str), kwargs=F(dict), milestones=F(list))

NATIVE_GEN = dict(tensor_parallel_size=F(int), pipeline_parallel_size=F(int), expert_parallel_size=F(int), gpu_memory_utilization=F(float, int),
                  max_model_len=F(int), block_size=F(int), kv_cache_tokens=F(int), max_running=F(int), use_cuda_graphs=F(bool),
                  enforce_eager=F(bool), precision=F(str, choices=("bfloat16", "bf16", "fp8", "mxfp8")), async_engine=F(bool),
                  decode_window=F(int), kv_block_size=F(int), enable_prefix_caching=F(bool), enable_chunked_prefill=F(bool), max_prefill_tokens=F(int),
                  kv_cache_dtype=F(str), skip_tokenizer_init=F(bool), load_format=F(str), hf_overrides=F(dict), use_deep_gemm=F(bool),
                  num_last_layers_in_bf16=F(int), num_first_layers_in_bf16=F(int), expose_http_server=F(bool), http_server_serving_chat_kwargs=F(dict),
                  enable_vllm_metrics_logger=F(bool), vllm_metrics_logger_interval=F(float, int), enable_expert_parallel=F(bool),
                  distributed_executor_backend=F(str), max_num_seqs=F(int), max_num_batched_tokens=F(int), vllm_kwargs=F(dict),
                  logprobs_mode=F(str), use_tqdm=F(bool), http_refit_api_key_env_var=F(str), reset_encoder_cache_after_weight_update=F(bool),
                  http_refit_server_port=F(int), zmq_refit_server_port=F(int))

COLOCATED = dict(enabled=F(bool, nullable=False), resources=F(dict, sub=dict(gpus_per_node=F(int), num_nodes=F(int))))

GENERATION = dict(backend=F(str, choices=("native", "vllm", "sglang", "megatron", "dynamo", "trtllm")), max_new_tokens=F(int), temperature=F(float, int),
                  top_p=F(float, int), top_k=F(int), stop_token_ids=F(list), stop_strings=F(list), model_name=F(str),
                  block_size=F(int), gpu_memory_utilization=F(float, int), kv_cache_tokens=F(int), max_model_len=F(int), max_running=F(int),
                  max_prefill_tokens=F(int), use_cuda_graphs=F(bool), free_kv_cache_on_sleep=F(bool), seed=F(int),
                  precision=F(str, choices=("bfloat16", "bf16", "fp8", "mxfp8")), decode_window=F(int),
                  native_cfg=F(dict, sub=NATIVE_GEN), vllm_cfg=F(dict, sub=NATIVE_GEN), sglang_cfg=OPAQUE, mcore_generation_config=OPAQUE,
                  colocated=F(dict, sub=COLOCATED), vllm_kwargs=F(dict), pad_token_id=F(int), _pad_token_id=F(int),
                  port_range_low=F(int), port_range_high=F(int), val_temperature=F(float, int), val_top_p=F(float, int), val_top_k=F(int),
                  refit_transport=F(str), real_quant_export_cpu_offload=F(bool), refit_cfg=F(dict))

# draft head trained beside the policy (nemo_rl/models/policy/__init__.py:497 DraftConfig)
DRAFT = dict(enabled=F(bool, nullable=False), model_name=F(str), loss_weight=F(float, int), num_layers=F(int), aux_layer_indices=F(list),
             draft_vocab_size=F(int))

POLICY = dict(
    model_name=F(str), tokenizer=F(dict, sub=TOKENIZER), train_global_batch_size=F(int, required=True, nullable=False),
    train_micro_batch_size=F(int, required=True, nullable=False), logprob_batch_size=F(int), logprob_chunk_size=F(int),
    generation=F(dict, sub=GENERATION), generation_batch_size=F(int), precision=F(str, choices=("bfloat16", "float32", "float16", "bf16", "fp32")),
    reward_model_cfg=F(dict), dtensor_cfg=F(dict, sub=DTENSOR), megatron_cfg=F(dict, sub=MEGATRON), draft=F(dict, sub=DRAFT),
    pretrained_checkpoint=F(dict), router_replay=F(dict, sub=dict(enabled=F(bool))), hf_config_overrides=F(dict),
    dynamic_batching=F(dict, sub=DYNAMIC_BATCHING), sequence_packing=F(dict, sub=PACKING), make_sequence_length_divisible_by=F(int),
    max_total_sequence_length=F(int, required=True, nullable=False), max_grad_norm=F(float, int), refit_buffer_size_gb=F(float, int),
    optimizer=F(dict, sub=OPTIMIZER), scheduler=F(list, dict, item=SCHEDULER_ITEM), quant_cfg=F(str), quant_calib_data=F(str),
    quant_calib_size=F(int), quant_batch_size=F(int), quant_sequence_length=F(int), disable_modelopt_layer_spec=F(bool), is_vlm=F(bool),
    # keys of this framework
    parallel=F(dict, sub=PARALLEL), activation_checkpointing=F(bool), grad_dtype=F(str, choices=("float32", "bfloat16")),
    offload_optimizer_for_logprob=F(bool), fused_optimizer=F(bool), fused_tensor_parallel=F(bool), fused_expert_parallel=F(bool),
    peer_wait_limit_s=F(float, int), lora_cfg=F(dict, sub=LORA), peft=F(dict, sub=LORA), fp8_cfg=F(dict, sub=FP8),
    offload_optimizer_states=F(bool), fsdp_offload_enabled=F(bool), model_cfg=F(dict), value_head=F(bool), temperature=F(float, int),
    top_k=F(int), top_p=F(float, int), algorithm=F(str), use_fused_lm_head=F(bool), seed=F(int),
)

LOSS_CLIPPED_PG = dict(
    disable_ppo_ratio=F(bool), token_level_loss=F(bool), sequence_level_importance_ratios=F(bool), ratio_clip_min=F(float, int, nullable=False),
    ratio_clip_max=F(float, int, nullable=False), ratio_clip_c=F(float, int), reference_policy_kl_penalty=F(float, int, nullable=False),
    reference_policy_kl_type=F(str, choices=("k1", "k2", "k3")), kl_input_clamp_value=F(float, int), kl_output_clamp_value=F(float, int),
    use_kl_in_reward=F(bool), use_importance_sampling_correction=F(bool),
    truncated_importance_sampling_type=F(str, choices=("tis", "icepop", "seq-mask-tis")), truncated_importance_sampling_ratio=F(float, int),
    truncated_importance_sampling_ratio_min=F(float, int), use_on_policy_kl_approximation=F(bool), force_on_policy_ratio=F(bool),
    use_cispo=F(bool), positive_example_nll_weight=F(float, int), ratio_clip_value=F(float, int), entropy_bonus=F(float, int),
)

ADV_ESTIMATOR = dict(name=F(str, choices=("grpo", "gdpo", "reinforce_plus_plus", "raw", "gae", "opd")), normalize_rewards=F(bool),
                     use_leave_one_out_baseline=F(bool), minus_baseline=F(bool), reward_weights=F(list), kl_reward_to_go=F(bool),
                     normalize_advantages=F(bool), gamma=F(float, int), gae_lambda=F(float, int), lambda_critic=F(float, int),
                     length_adaptive_alpha=F(float, int))
ADV_ESTIMATOR["lambda"] = F(float, int)

ASYNC_GRPO = dict(enabled=F(bool), max_trajectory_age_steps=F(int), in_flight_weight_updates=F(bool), recompute_kv_cache_after_weight_updates=F(bool),
                  train_ranks=F(int), generation_ranks=F(int), replay_buffer_capacity=F(int), max_generation_failures=F(int))

GRPO = dict(
    num_prompts_per_step=F(int, nullable=False), num_generations_per_prompt=F(int, nullable=False), max_num_epochs=F(int), max_num_steps=F(int),
    max_rollout_turns=F(int), normalize_rewards=F(bool), advantage_clip_low=F(float, int), advantage_clip_high=F(float, int),
    use_leave_one_out_baseline=F(bool), val_period=F(int), val_start_at=F(int), val_batch_size=F(int), val_at_start=F(bool), val_at_end=F(bool),
    max_val_samples=F(int), val_num_generations_per_prompt=F(int), stop_at_validation_metric=F(str), stop_at_validation_threshold=F(float, int),
    skip_reference_policy_logprobs_calculation=F(bool), seed=F(int), async_grpo=F(dict, sub=ASYNC_GRPO), overlong_filtering=F(bool),
    use_dynamic_sampling=F(bool), dynamic_sampling_max_gen_batches=F(int), batch_multiplier=F(float, int), reward_shaping=F(dict),
    reward_scaling=F(dict), calculate_advantages_on_gpu=F(bool), seq_logprob_error_threshold=F(float, int),
    invalid_tool_call_advantage=F(float, int), malformed_thinking_advantage=F(float, int), adv_estimator=F(dict, sub=ADV_ESTIMATOR),
    deduplicate_multimodal_data=F(bool), debug_payload_metrics=F(bool),
)

CHECKPOINTING = dict(enabled=F(bool, nullable=False), checkpoint_dir=F(str), metric_name=F(str), higher_is_better=F(bool), keep_top_k=F(int),
                     save_period=F(int), checkpoint_must_save_by=F(str), model_save_format=F(str, choices=("safetensors", "torch_save", "dcp")),
                     save_consolidated=F(bool), save_optimizer=F(bool), ft_save_period=F(int), ft_keep_latest_k=F(int),
                     model_cache_dir=F(str), model_repo_id=F(str), is_peft=F(bool), peft_config=F(dict))

LOGGER = dict(log_dir=F(str), wandb_enabled=F(bool), tensorboard_enabled=F(bool), mlflow_enabled=F(bool), swanlab_enabled=F(bool),
              monitor_gpus=F(bool), num_val_samples_to_print=F(int), wandb=F(dict), tensorboard=F(dict), mlflow=F(dict), swanlab=F(dict),
              gpu_monitoring=F(dict, sub=dict(collection_interval=F(float, int), flush_interval=F(float, int))))

CLUSTER = dict(gpus_per_node=F(int, nullable=False), num_nodes=F(int, nullable=False), segment_size=F(int), master_port_range_low=F(int),
               master_port_range_high=F(int), backend=F(str))

DATA = dict(max_input_seq_length=F(int), prompt_file=F(str), system_prompt_file=F(str), shuffle=F(bool), num_workers=F(int),
            dataset_name=F(str), add_bos=F(bool), add_eos=F(bool), add_generation_prompt=F(bool), train=F(dict, list), validation=F(dict, list),
            default=OPAQUE, seed=F(int), split=F(str), input_key=F(str), output_key=F(str), prompt_key=F(str), val_split=F(str),
            num_samples=F(int), use_multiple_dataloader=F(bool), num_prompts_per_dataloader=F(int), custom_dataloader=F(str), train_data_path=F(str),
            val_data_path=F(str), subset=F(str), filter_long_samples=F(bool), env_name=F(str), processor=F(str), batch_size=F(int))

SFT = dict(max_num_epochs=F(int), max_num_steps=F(int), val_period=F(int), val_batches=F(int), val_global_batch_size=F(int),
           val_micro_batch_size=F(int), val_at_start=F(bool), val_at_end=F(bool), seed=F(int), only_unmask_final=F(bool))

DPO = dict(SFT, reference_policy_kl_penalty=F(float, int), preference_average_log_probs=F(bool), sft_average_log_probs=F(bool),
           preference_loss_weight=F(float, int), sft_loss_weight=F(float, int))

PPO = dict(GRPO, critic=F(dict), gamma=F(float, int), value_clip=F(float, int), critic_warmup_steps=F(int), vapo=F(dict),
           gae_lambda=F(float, int), lambda_critic=F(float, int), length_adaptive_alpha=F(float, int), normalize_advantages=F(bool),
           num_value_warmup_steps=F(int), policy_epochs=F(int), value_epochs=F(int), ppo_epochs=F(int), policy_training_start_step=F(int),
           async_ppo=F(dict))
PPO["lambda"] = F(float, int)

DISTILLATION = dict(num_prompts_per_step=F(int), num_generations_per_prompt=F(int), max_rollout_turns=F(int), max_num_steps=F(int),
                    max_num_epochs=F(int), val_period=F(int), val_batch_size=F(int), val_at_start=F(bool), val_at_end=F(bool),
                    max_val_samples=F(int), topk_logits_k=F(int), seed=F(int), text_key=F(str))

# a policy section that only serves or scores (teacher, evaluation): the batch-size keys are optional
POLICY_INFERENCE = {k: (Field(v.types, False, v.nullable, v.choices, v.sub, v.item, v.doc) if v.required else v) for k, v in POLICY.items()}

EVAL = dict(metric=F(str), num_tests_per_prompt=F(int), seed=F(int), k_value=F(int), save_path=F(str), pass_k_value=F(int))

# top-level section -> schema, per algorithm
_SECTIONS = {
    "grpo": dict(policy=POLICY, loss_fn=LOSS_CLIPPED_PG, grpo=GRPO, checkpointing=CHECKPOINTING, logger=LOGGER, cluster=CLUSTER, data=DATA),
    "sft": dict(policy=POLICY, sft=SFT, checkpointing=CHECKPOINTING, logger=LOGGER, cluster=CLUSTER, data=DATA),
    "dpo": dict(policy=POLICY, dpo=DPO, sft=SFT, checkpointing=CHECKPOINTING, logger=LOGGER, cluster=CLUSTER, data=DATA),
    "rm": dict(policy=POLICY, rm=SFT, sft=SFT, checkpointing=CHECKPOINTING, logger=LOGGER, cluster=CLUSTER, data=DATA),
    "ppo": dict(policy=POLICY, value=POLICY_INFERENCE, loss_fn=LOSS_CLIPPED_PG, ppo=PPO, grpo=GRPO, checkpointing=CHECKPOINTING, logger=LOGGER, cluster=CLUSTER, data=DATA),
    "eval": dict(policy=POLICY_INFERENCE, generation=GENERATION, eval=EVAL, logger=LOGGER, cluster=CLUSTER, data=DATA),
    "distillation": dict(policy=POLICY, teacher=POLICY_INFERENCE, distillation=DISTILLATION, grpo=GRPO, checkpointing=CHECKPOINTING, logger=LOGGER,
                         cluster=CLUSTER, data=DATA),
}
_TOP_LEVEL_FREE = ("env", "defaults", "env_vars", "data_plane", "reward_penalties", "on_policy_distillation", "eval", "generation",
                   "tokenizer", "async_rl", "single_controller", "loss_fn", "teacher", "critic", "profiling")

_reported: set = set()


def validate_master_config(cfg: dict, algorithm: str = "grpo", *, strict: bool = False, quiet: bool = False) -> Report:
    """Validates a whole recipe. Errors raise ``ConfigError``; unknown keys are printed once per process (``strict``
    turns them into errors too). Returns the report."""
    sections = _SECTIONS.get(algorithm)
    if sections is None:
        raise ConfigError(f"no schema for algorithm '{algorithm}' (known: {sorted(_SECTIONS)})")
    rep = Report()
    for name, schema in sections.items():
        if name in cfg:
            validate(name, cfg[name], schema, rep)
    for k in cfg:
        if k not in sections and k not in _TOP_LEVEL_FREE:
            close = difflib.get_close_matches(str(k), list(sections) + list(_TOP_LEVEL_FREE), n=1, cutoff=0.75)
            rep.unknown.append((str(k), close[0] if close else None))
    if strict and rep.unknown:
        rep.errors.extend(f"unknown key {p}" + (f" (did you mean '{h}'?)" if h else "") for p, h in rep.unknown)
    if rep.errors:
        raise ConfigError("configuration did not validate:\n" + rep.render())
    fresh = [(p, h) for p, h in rep.unknown if p not in _reported]
    if fresh and not quiet:
        _reported.update(p for p, _ in fresh)
        print("[config] keys that no component of this framework reads (listed once):")
        for p, h in fresh:
            print(f"[config]   {p}" + (f"   <- did you mean '{h}'?" if h else ""))
    return rep


def policy_config(cfg: dict) -> dict:
    """Validates one policy section on its own (workers built outside an entry point)."""
    rep = validate("policy", cfg, POLICY)
    if rep.errors:
        raise ConfigError("policy configuration did not validate:\n" + rep.render())
    return cfg
