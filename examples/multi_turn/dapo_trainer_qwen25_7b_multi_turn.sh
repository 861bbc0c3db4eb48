#!/bin/bash
# DAPO with multi-turn tool calls in the rollout (tools from configs/tools).
# Usage: bash examples/multi_turn/dapo_trainer_qwen25_7b_multi_turn.sh [recipe name without .yaml] [key=value overrides ...]
source "$(dirname "$0")/../common.sh"
launch_trainer train_dapo.py dapo_qwen25_7b_multi_turn_b200 "$@"
