#!/bin/bash
# GRPO with rollout routing replay on a model with experts.
source "$(dirname "$0")/common.sh"
run_and_check grpo_router_replay "$PY" examples/run_grpo.py --config examples/configs/grpo_arithmetic_offline.yaml grpo.max_num_steps=2 \
  policy.model_name=tiny-nemotron-h +policy.router_replay.enabled=true -- 'max(data["train/token_mult_prob_error"]) < 1.05'
