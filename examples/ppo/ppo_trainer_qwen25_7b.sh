#!/bin/bash
# PPO with a critic, Qwen2.5-7B.
# Usage: bash examples/ppo/ppo_trainer_qwen25_7b.sh [recipe name without .yaml] [key=value overrides ...]
source "$(dirname "$0")/../common.sh"
launch_trainer train_ppo.py ppo_qwen25_7b_b200 "$@"
