#!/usr/bin/env python
"""Convert checkpoints between the Hugging Face layout and the mcore ``torch`` layout.

    python cli/convert_ckpt.py hf2mcore --model qwen25_7b --load ./Qwen2.5-7B --save ./ckpt --tp 4 --pp 1
    python cli/convert_ckpt.py mcore2hf --model qwen25_7b --load ./ckpt --save ./hf_out --tp 4 --pp 1
    (MoE: add --ep N and --moe-tp-extend-ep; reward / critic heads: --orm)
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..")))

from mindspeed_rl_b200.checkpoint import convert as C  # noqa: E402
from mindspeed_rl_b200.config import MegatronConfig  # noqa: E402
from mindspeed_rl_b200.config.loader import load_model_catalogue  # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("direction", choices=["hf2mcore", "mcore2hf"])
    ap.add_argument("--model", required=True, help="name of a configs/model/<name>.yaml architecture")
    ap.add_argument("--load", required=True)
    ap.add_argument("--save", required=True)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--ep", type=int, default=1)
    ap.add_argument("--moe-tp-extend-ep", action="store_true")
    ap.add_argument("--num-layer-list", default=None, help="comma separated layers per pipeline stage")
    ap.add_argument("--orm", action="store_true")
    a = ap.parse_args(argv)
    cfg = MegatronConfig({"model": a.model}, load_model_catalogue([a.model]))
    cfg.num_query_groups = cfg.num_query_groups if cfg.group_query_attention else cfg.num_attention_heads
    nll = [int(x) for x in a.num_layer_list.split(",")] if a.num_layer_list else None
    if a.direction == "hf2mcore":
        shards = C.hf_to_mcore(C.load_hf_state(a.load), cfg, a.tp, a.pp, a.ep, a.moe_tp_extend_ep, nll, a.orm)
        C.write_mcore(shards, a.save, a.tp, a.pp, a.ep, args={"model": a.model, "tp": a.tp, "pp": a.pp, "ep": a.ep})
    else:
        hf = C.mcore_to_hf(C.read_mcore(a.load, a.tp, a.pp, a.ep), cfg, a.tp, a.pp, a.ep, a.moe_tp_extend_ep, nll)
        C.save_hf_state(hf, a.save)
    print(f"{a.direction}: wrote {a.save}")


if __name__ == "__main__":
    main()
