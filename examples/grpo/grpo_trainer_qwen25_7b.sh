#!/bin/bash
# GRPO, Qwen2.5-7B, one 8-GPU node: train TP4 x DP2, rollout TP2 x DP4, co-located.
# Usage: bash examples/grpo/grpo_trainer_qwen25_7b.sh [recipe name without .yaml] [key=value overrides ...]
source "$(dirname "$0")/../common.sh"
launch_trainer train_grpo.py grpo_qwen25_7b_b200 "$@"
