#!/bin/bash
# DPO on pairwise preference data, Qwen3-30B-A3B.
# Usage: bash examples/dpo/dpo_trainer_qwen3_30b_a3b.sh [recipe name without .yaml] [key=value overrides ...]
source "$(dirname "$0")/../common.sh"
launch_trainer train_dpo.py dpo_qwen3_30b_a3b_b200 "$@"
