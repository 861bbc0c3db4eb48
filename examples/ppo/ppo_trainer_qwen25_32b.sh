#!/bin/bash
# PPO, Qwen2.5-32B: actor + critic + frozen reference co-located, Adam state in pinned host memory.
# Usage: bash examples/ppo/ppo_trainer_qwen25_32b.sh [recipe name without .yaml] [key=value overrides ...]
source "$(dirname "$0")/../common.sh"
launch_trainer train_ppo.py ppo_qwen25_32b_b200 "$@"
