#!/bin/bash
# DAPO (clip-higher, dynamic sampling, token-level loss), Qwen2.5-7B.
# Usage: bash examples/dapo/dapo_trainer_qwen25_7b.sh [recipe name without .yaml] [key=value overrides ...]
source "$(dirname "$0")/../common.sh"
launch_trainer train_dapo.py dapo_qwen25_7b_b200 "$@"
