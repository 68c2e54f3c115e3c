#!/bin/bash
# GRPO with a draft head trained along: its loss is logged beside the policy's.
source "$(dirname "$0")/common.sh"
run_and_check grpo_draft "$PY" examples/run_grpo.py --config examples/configs/grpo_arithmetic_offline.yaml grpo.max_num_steps=2 \
  +policy.draft.enabled=true -- 'max(data["train/token_mult_prob_error"]) < 1.05' 'min(data["train/draft_loss"]) > 0'
