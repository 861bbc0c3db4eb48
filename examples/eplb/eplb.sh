#!/bin/bash
# Turn the collected expert-load statistics into a placement map with redundant experts.
# Usage: bash examples/eplb/eplb.sh <dump dir> <output map.json> <rollout GPUs> [redundant expert slots per GPU]
set -euo pipefail
ROOT=$(cd "$(dirname "$0")/../.." && pwd)
export PYTHONPATH="$ROOT:${PYTHONPATH:-}"
DUMP_DIR=${1:?dump directory}
OUT=${2:?output json}
EP=${3:?number of rollout GPUs}
REDUNDANT=${4:-0}
python "$ROOT/cli/eplb_generate_map.py" --json_folder "$DUMP_DIR" --output "$OUT" --num_gpus "$EP" --num_redundancy "$REDUNDANT"
