#!/bin/bash
# Tokenise a JSON / parquet dataset into the indexed .bin/.idx files the trainers read.
# Usage: bash examples/data/preprocess_data.sh [dataset config name under configs/datasets, default: math_17k]
set -euo pipefail
ROOT=$(cd "$(dirname "$0")/../.." && pwd)
export PYTHONPATH="$ROOT:${PYTHONPATH:-}"
python "$ROOT/cli/preprocess_data.py" "${1:-math_17k}"
