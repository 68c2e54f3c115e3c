#!/bin/bash
# Vision-language GRPO on synthetic images, two steps.
source "$(dirname "$0")/common.sh"
run_and_check vlm_grpo "$PY" examples/run_vlm_grpo.py --config examples/configs/vlm_grpo_offline.yaml grpo.max_num_steps=2 -- \
  'max(data["train/token_mult_prob_error"]) < 1.05' 'len(data["train/loss"]) == 2'
