#!/bin/bash
# DAPO, Qwen2.5-32B, 32k context (context parallel + remove-padding token budgets).
# Usage: bash examples/dapo/dapo_trainer_qwen25_32b_32k.sh [recipe name without .yaml] [key=value overrides ...]
source "$(dirname "$0")/../common.sh"
launch_trainer train_dapo.py dapo_qwen25_32b_32k_b200 "$@"
