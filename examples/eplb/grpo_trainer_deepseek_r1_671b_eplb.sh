#!/bin/bash
# GRPO with an expert-placement map produced by examples/eplb/eplb.sh (recipe key generate_config.expert_map_path).
# Usage: bash examples/eplb/grpo_trainer_deepseek_r1_671b_eplb.sh [recipe name without .yaml] [key=value overrides ...]
source "$(dirname "$0")/../common.sh"
launch_trainer train_grpo.py grpo_deepseek_r1_671b_eplb_b200 "$@"
