#!/bin/bash
# GRPO, Qwen2.5-32B (two nodes in the shipped recipe: set NNODES / NODE_RANK / MASTER_ADDR).
# Usage: bash examples/grpo/grpo_trainer_qwen25_32b_1k.sh [recipe name without .yaml] [key=value overrides ...]
source "$(dirname "$0")/../common.sh"
launch_trainer train_grpo.py grpo_qwen25_32b_1k_b200 "$@"
