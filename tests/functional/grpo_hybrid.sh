#!/bin/bash
# GRPO on the hybrid Mamba-2 / attention / MLP / expert model: engine state pools and trainer scan agree.
source "$(dirname "$0")/common.sh"
run_and_check grpo_hybrid "$PY" examples/run_grpo.py --config examples/configs/grpo_arithmetic_offline.yaml grpo.max_num_steps=2 \
  policy.model_name=tiny-nemotron-h -- 'max(data["train/token_mult_prob_error"]) < 1.05' 'len(data["train/loss"]) == 2'
