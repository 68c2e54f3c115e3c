#!/bin/bash
# GRPO, 3 steps on the offline arithmetic recipe: the two halves of the step agree and the phases are all timed.
source "$(dirname "$0")/common.sh"
run_and_check grpo "$PY" examples/run_grpo.py --config examples/configs/grpo_arithmetic_offline.yaml grpo.max_num_steps=3 -- \
  'max(data["train/token_mult_prob_error"]) < 1.05' 'max(data["train/gen_kl_error"]) < 0.002' 'len(data["train/loss"]) == 3' \
  'min(data["timing/train/generation"]) > 0' 'min(data["timing/train/policy_training"]) > 0'
