#!/bin/bash
# DAPO, Qwen3-32B.
# Usage: bash examples/dapo/dapo_trainer_qwen3_32b.sh [recipe name without .yaml] [key=value overrides ...]
source "$(dirname "$0")/../common.sh"
launch_trainer train_dapo.py dapo_qwen3_32b_b200 "$@"
