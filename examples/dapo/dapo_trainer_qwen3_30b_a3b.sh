#!/bin/bash
# DAPO, Qwen3-30B-A3B mixture of experts, expert parallel 8.
# Usage: bash examples/dapo/dapo_trainer_qwen3_30b_a3b.sh [recipe name without .yaml] [key=value overrides ...]
source "$(dirname "$0")/../common.sh"
launch_trainer train_dapo.py dapo_qwen3_30b_a3b_b200 "$@"
