# Shared by the functional scripts: every script runs ONE entrypoint for a few steps on the offline recipes (CPU or one GPU),
# dumps the logged metrics and asserts on them.  Usage inside a script:
#   source "$(dirname "$0")/common.sh"; run_and_check <name> <command...> -- <check expressions...>
set -euo pipefail
ROOT="$(cd "$(dirname "${BASH_SOURCE[0]}")/../.." && pwd)"
OUT="${RLB_FUNCTIONAL_OUT:-/tmp/rlb_functional}"
PY="${PYTHON:-python}"
export OMP_NUM_THREADS="${OMP_NUM_THREADS:-4}"

run_and_check() {
  local name="$1"; shift
  local cmd=() checks=() seen_sep=0
  for a in "$@"; do
    if [ "$a" = "--" ] && [ $seen_sep -eq 0 ]; then seen_sep=1; continue; fi
    if [ $seen_sep -eq 0 ]; then cmd+=("$a"); else checks+=("$a"); fi
  done
  local dir="$OUT/$name"
  rm -rf "$dir"; mkdir -p "$dir"
  ( cd "$ROOT" && "${cmd[@]}" "logger.log_dir=$dir/logs" "checkpointing.checkpoint_dir=$dir/ckpt" ) > "$dir/run.log" 2>&1 \
    || { tail -40 "$dir/run.log"; echo "FAILED: $name (run)"; return 1; }
  "$PY" "$ROOT/tests/json_dump_metrics.py" "$dir/logs" --output_path "$dir/metrics.json" > /dev/null
  "$PY" "$ROOT/tests/check_metrics.py" "$dir/metrics.json" "${checks[@]}" || { echo "FAILED: $name (metrics)"; return 1; }
  echo "OK: $name"
}
