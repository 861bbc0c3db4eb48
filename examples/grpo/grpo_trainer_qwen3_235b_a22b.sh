#!/bin/bash
# GRPO, Qwen3-235B-A22B mixture of experts (multi-node: expert parallel training and rollout).
# Usage: bash examples/grpo/grpo_trainer_qwen3_235b_a22b.sh [recipe name without .yaml] [key=value overrides ...]
source "$(dirname "$0")/../common.sh"
launch_trainer train_grpo.py grpo_qwen3_235b_a22b_b200 "$@"
