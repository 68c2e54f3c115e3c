#!/bin/bash
# Cross-tokenizer off-policy distillation (byte student, byte-pair teacher), two steps.
source "$(dirname "$0")/common.sh"
run_and_check xtoken_distillation "$PY" examples/run_xtoken_off_policy_distillation.py --config examples/configs/xtoken_distillation_offline.yaml \
  distillation.max_num_steps=2 data.num_samples=32 -- 'len(data["train/loss"]) == 2' 'min(data["train/aligned_positions"]) > 0'
