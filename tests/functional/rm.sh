#!/bin/bash
# Bradley-Terry reward model, two steps on random preference pairs.
source "$(dirname "$0")/common.sh"
run_and_check rm "$PY" examples/run_rm.py --config examples/configs/rm.yaml policy.model_name=tiny-llama-oracle policy.tokenizer.name=byte policy.max_total_sequence_length=64 policy.train_global_batch_size=8 policy.train_micro_batch_size=4 policy.scheduler=null logger.monitor_gpus=false policy.sequence_packing.sequence_length_round=1 rm.max_num_steps=2 rm.val_period=0 \
  rm.val_at_start=false data.train.dataset_name=random_preference data.validation.dataset_name=random_preference -- \
  'len(data["train/loss"]) == 2' 'max(data["train/loss"]) < 5'
