#!/bin/bash
# GRPO with LoRA adapters on Qwen2.5-32B (the frozen backbone is the reference policy).
# Usage: bash examples/grpo/grpo_trainer_lora_qwen25_32b.sh [recipe name without .yaml] [key=value overrides ...]
source "$(dirname "$0")/../common.sh"
launch_trainer train_grpo.py grpo_lora_qwen25_32b_b200 "$@"
