#!/bin/bash
# SFT, a few steps on random data: the loss is finite and falls (the model memorises the batch distribution's unigram statistics).
source "$(dirname "$0")/common.sh"
run_and_check sft "$PY" examples/run_sft.py --config examples/configs/sft.yaml policy.model_name=tiny-llama-oracle policy.tokenizer.name=byte policy.max_total_sequence_length=64 policy.train_global_batch_size=8 policy.train_micro_batch_size=4 policy.scheduler=null logger.monitor_gpus=false policy.sequence_packing.sequence_length_round=1 sft.max_num_steps=6 sft.val_period=0 \
  sft.val_at_start=false data.train.dataset_name=random_sft data.validation.dataset_name=random_sft -- \
  'len(data["train/loss"]) == 6' 'max(data["train/loss"]) < 20' 'last(data["train/loss"]) <= first(data["train/loss"]) + 0.5'
