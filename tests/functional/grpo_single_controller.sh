#!/bin/bash
# Single-controller GRPO: rollout and train pumps over the data plane.
source "$(dirname "$0")/common.sh"
run_and_check grpo_single_controller "$PY" examples/run_grpo_single_controller.py --config examples/configs/grpo_single_controller.yaml \
  grpo.max_num_steps=2 -- 'len(data["train/loss"]) >= 2'
