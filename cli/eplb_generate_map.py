#!/usr/bin/env python
"""Build ``expert_map.json`` from the per-rank routing statistics a rollout run dumped.

    python cli/eplb_generate_map.py --json_folder ./eplb --num_gpus 8 [--num_redundancy 1] [--output expert_map.json]

Reads every ``eplb_token_collects_*.json`` (``{layer: {expert: count}}``), sums them into a
``[layers, experts]`` matrix, runs the load balancer and writes the placement the rollout engine
loads through ``generate_config.expert_map_path`` (reference: ``cli/eplb_generate_map_ds.py:13-191``).
"""
import argparse
import glob
import json
import os
import sys

import torch

sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..")))

from mindspeed_rl_b200.rollout.eplb import expert_map_from_counts  # noqa: E402


def load_counts(folder: str) -> torch.Tensor:
    files = sorted(glob.glob(os.path.join(folder, "eplb_token_collects_*.json")))
    if not files:
        raise FileNotFoundError(f"no eplb_token_collects_*.json under {folder}")
    total = None
    for f in files:
        data = json.load(open(f))
        layers = sorted(data, key=int)
        mat = torch.tensor([[data[l][e] for e in sorted(data[l], key=int)] for l in layers], dtype=torch.float64)
        total = mat if total is None else total + mat
    return total


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--json_folder", required=True)
    ap.add_argument("--num_gpus", type=int, required=True)
    ap.add_argument("--num_redundancy", type=int, default=1, help="redundant expert slots per GPU")
    ap.add_argument("--num_groups", type=int, default=1)
    ap.add_argument("--num_nodes", type=int, default=1)
    ap.add_argument("--output", default="expert_map.json")
    a = ap.parse_args(argv)
    emap = expert_map_from_counts(load_counts(a.json_folder), a.num_gpus, a.num_redundancy, a.num_groups, a.num_nodes)
    with open(a.output, "w") as fh:
        json.dump(emap, fh, indent=1)
    print(f"wrote {a.output}: {emap['moe_layer_count']} layers x {a.num_gpus} devices")


if __name__ == "__main__":
    main()
