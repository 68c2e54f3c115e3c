#!/bin/bash
# Runs ONE recipe of examples/configs/recipes for a few steps and asserts on its logged metrics (the role of the reference's
# per-recipe scripts under tests/test_suites/{llm,vlm}/, which this repository keeps as lines of the suite lists instead).
#
#   tests/test_suites/run_recipe.sh <recipe.yaml relative to examples/configs/recipes> [steps]
#
# The entrypoint is chosen from the recipe's algorithm section; the number of ranks from its cluster section (torchrun when > 1).
# Set NUM_NODES / GPUS_PER_NODE to override the cluster size, EXTRA_OVERRIDES for additional `key=value` overrides, and
# PRESET=<preset name> to run a preset architecture with random weights and the byte tokenizer instead of the recipe's
# HuggingFace checkpoint (no download; for smoke runs).
set -euo pipefail
ROOT="$(cd "$(dirname "$0")/../.." && pwd)"
RECIPE="$1"; STEPS="${2:-10}"
NAME="$(basename "${RECIPE%.yaml}")"
OUT="${RLB_SUITE_OUT:-$ROOT/results/test_suites}/$NAME"
mkdir -p "$OUT"
read -r ALGO ENTRY GPUS NODES <<<"$(python - "$ROOT/examples/configs/recipes/$RECIPE" <<'PY'
import sys
sys.path.insert(0, sys.argv[1].split("/examples/")[0])
from rl_b200.utils.config import load_config
from rl_b200.utils.cli import infer_algorithm
cfg = load_config(sys.argv[1])
algo = infer_algorithm(cfg)
entry = {"grpo": "run_grpo.py", "sft": "run_sft.py", "dpo": "run_dpo.py", "rm": "run_rm.py", "ppo": "run_ppo.py", "distillation": "run_distillation.py",
         "eval": "run_eval.py"}[algo]
if "vlm" in sys.argv[1]:
    entry = "run_vlm_grpo.py" if algo == "grpo" else "run_vlm_sft.py"
c = cfg.get("cluster") or {}
print(algo, entry, int(c.get("gpus_per_node", 1)), int(c.get("num_nodes", 1)))
PY
)"
GPUS="${GPUS_PER_NODE:-$GPUS}"; NODES="${NUM_NODES:-$NODES}"
OVERRIDES=("$ALGO.max_num_steps=$STEPS" "logger.log_dir=$OUT/logs" "checkpointing.checkpoint_dir=$OUT/ckpt")
if [ -n "${PRESET:-}" ]; then OVERRIDES+=("policy.model_name=$PRESET" "policy.tokenizer.name=byte"); fi
OVERRIDES+=(${EXTRA_OVERRIDES:-})
cd "$ROOT"
if [ "$((GPUS * NODES))" -gt 1 ]; then
  LAUNCH=(python -m torch.distributed.run --nnodes="$NODES" --nproc-per-node "$GPUS" --master-addr "${MASTER_ADDR:-127.0.0.1}" --master-port "${MASTER_PORT:-29500}")
else
  LAUNCH=(python)
fi
"${LAUNCH[@]}" "examples/$ENTRY" --config "examples/configs/recipes/$RECIPE" "${OVERRIDES[@]}" 2>&1 | tee "$OUT/run.log"
python tests/json_dump_metrics.py "$OUT/logs" --output_path "$OUT/metrics.json"
CHECKS=("len(data[\"train/loss\"]) == $STEPS")
if [ "$ALGO" = "grpo" ]; then CHECKS+=('max(data["train/token_mult_prob_error"]) < 1.1' 'mean(data["timing/train/total_step_time"], 2) > 0'); fi
python tests/check_metrics.py "$OUT/metrics.json" "${CHECKS[@]}"
