#!/bin/bash
# GRPO from one controller process over two worker processes (worker groups + driver-side policy).
source "$(dirname "$0")/common.sh"
run_and_check grpo_controller "$PY" examples/run_grpo_controller.py --config examples/configs/grpo_arithmetic_offline.yaml grpo.max_num_steps=2 \
  cluster.gpus_per_node=2 +cluster.backend=gloo -- 'max(data["train/token_mult_prob_error"]) < 1.05' 'len(data["train/loss"]) == 2'
