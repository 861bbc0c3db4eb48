#!/bin/bash
# DAPO, Qwen2.5-32B, 20k responses (context parallel + remove-padding token budgets).
# Usage: bash examples/dapo/dapo_trainer_qwen25_32b_20k.sh [recipe name without .yaml] [key=value overrides ...]
source "$(dirname "$0")/../common.sh"
launch_trainer train_dapo.py dapo_qwen25_32b_20k_b200 "$@"
