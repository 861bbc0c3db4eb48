#!/bin/bash
# GRPO, Qwen3-8B with QK-RMSNorm.
# Usage: bash examples/grpo/grpo_trainer_qwen3_8b.sh [recipe name without .yaml] [key=value overrides ...]
source "$(dirname "$0")/../common.sh"
launch_trainer train_grpo.py grpo_qwen3_8b_b200 "$@"
