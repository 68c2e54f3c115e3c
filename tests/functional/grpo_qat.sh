#!/bin/bash
# Quantisation-aware GRPO (NVFP4 weights and inputs): engine and trainer see the same quantised policy.
source "$(dirname "$0")/common.sh"
run_and_check grpo_qat "$PY" examples/run_grpo.py --config examples/configs/grpo_arithmetic_offline.yaml grpo.max_num_steps=2 \
  +policy.quant_cfg=NVFP4_DEFAULT_CFG +policy.quant_calib_size=8 +policy.quant_sequence_length=32 -- \
  'max(data["train/token_mult_prob_error"]) < 1.05'
