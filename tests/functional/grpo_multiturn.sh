#!/bin/bash
# Multi-turn GRPO on the sliding puzzle environment.
source "$(dirname "$0")/common.sh"
run_and_check grpo_multiturn "$PY" examples/run_grpo_sliding_puzzle.py --config examples/configs/grpo_sliding_puzzle.yaml grpo.max_num_steps=2 \
  policy.model_name=tiny-llama-oracle policy.tokenizer.name=byte policy.max_total_sequence_length=256 policy.train_global_batch_size=8 \
  policy.train_micro_batch_size=4 policy.scheduler=null logger.monitor_gpus=false grpo.num_prompts_per_step=4 grpo.num_generations_per_prompt=2 \
  policy.generation.max_new_tokens=16 -- \
  'max(data["train/token_mult_prob_error"]) < 1.05' 'max(data["train/avg_turns_per_sample"]) >= 1'
