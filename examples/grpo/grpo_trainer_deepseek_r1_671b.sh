#!/bin/bash
# GRPO, DeepSeek-R1-671B (multi-latent attention, 256 routed experts; multi-node).
# Usage: bash examples/grpo/grpo_trainer_deepseek_r1_671b.sh [recipe name without .yaml] [key=value overrides ...]
source "$(dirname "$0")/../common.sh"
launch_trainer train_grpo.py grpo_deepseek_r1_671b_b200 "$@"
