#!/bin/bash
# GRPO on two data-parallel ranks (gloo on CPU, NCCL on GPUs).
source "$(dirname "$0")/common.sh"
run_and_check grpo_dp2 "$PY" -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port "${MASTER_PORT:-29611}" \
  examples/run_grpo.py --config examples/configs/grpo_arithmetic_offline.yaml grpo.max_num_steps=2 -- \
  'max(data["train/token_mult_prob_error"]) < 1.05' 'len(data["train/loss"]) == 2'
