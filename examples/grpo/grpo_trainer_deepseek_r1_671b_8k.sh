#!/bin/bash
# GRPO, DeepSeek-V3/R1 671B, 8k prompts, rollout TP4 x EP16.
# Usage: bash examples/grpo/grpo_trainer_deepseek_r1_671b_8k.sh [recipe name without .yaml] [key=value overrides ...]
source "$(dirname "$0")/../common.sh"
launch_trainer train_grpo.py grpo_deepseek_r1_671b_8k_b200 "$@"
