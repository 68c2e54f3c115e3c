#!/bin/bash
# Runs every functional script (CPU: a few minutes; one GPU: faster). A script that fails is reported and the run goes on.
cd "$(dirname "$0")"
failed=()
for s in grpo.sh grpo_hybrid.sh grpo_router_replay.sh grpo_qat.sh grpo_draft.sh grpo_controller.sh grpo_single_controller.sh grpo_multiturn.sh \
         grpo_dp2.sh sft.sh dpo.sh rm.sh xtoken_distillation.sh vlm_grpo.sh; do
  echo "=== $s"
  bash "./$s" || failed+=("$s")
done
if [ ${#failed[@]} -gt 0 ]; then echo "FAILED: ${failed[*]}"; exit 1; fi
echo "all functional scripts passed"
