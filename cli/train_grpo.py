#!/usr/bin/env python
"""GRPO training entry point.

    torchrun --nproc-per-node N cli/train_grpo.py --config-name <yaml stem> [--config-dir DIR] [section.key=value ...]

One process per GPU; the YAML schema (``megatron_training / actor_config / rl_config /
generate_config / ...``) is described in ``configs/``.  Reference entry point: ``cli/train_grpo.py``.
"""
import os
import sys

sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..")))

from mindspeed_rl_b200.runtime.launch import main  # noqa: E402

if __name__ == "__main__":
    main("grpo", default_config="grpo_qwen25_7b_b200")
