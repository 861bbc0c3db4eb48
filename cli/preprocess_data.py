#!/usr/bin/env python
"""Tokenise a raw dataset into packed ``.bin/.idx`` files.

    python cli/preprocess_data.py <dataset-yaml-stem> [--config-dir DIR] [key=value ...]

The YAML (``configs/datasets/<stem>.yaml``) holds the :class:`DataHandlerConfig` options:
``input``, ``tokenizer_name_or_path``, ``handler_name``, ``prompt_type``, ``output_prefix``,
``dataset_additional_keys``, ``map_keys`` ...  With ``n_subs > 1`` the input rows are split into
``n_subs`` parts that are tokenised by a process pool and merged afterwards.
(Reference entry point: ``cli/preprocess_data.py:79-165``.)
"""
import multiprocessing as mp
import os
import sys

import yaml

sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..")))

from mindspeed_rl_b200.config import DataHandlerConfig, DEFAULT_CONFIG_DIR, validate_data_handler_config  # noqa: E402
from mindspeed_rl_b200.config.loader import apply_overrides  # noqa: E402
from mindspeed_rl_b200.datasets.data_handler import build_dataset, get_dataset_handler  # noqa: E402
from mindspeed_rl_b200.datasets.indexed_dataset import (IndexedDatasetBuilder, _Index, get_bin_path,  # noqa: E402
                                                        get_idx_path)
from mindspeed_rl_b200.utils.tokenizer import get_tokenizer  # noqa: E402


def _load_config(argv):
    name, cfg_dir, overrides = None, None, []
    it = iter(argv)
    for a in it:
        if a in ("--config-dir", "-cd"):
            cfg_dir = next(it)
        elif "=" in a and not a.startswith("--"):
            overrides.append(a)
        elif name is None:
            name = a
    if name is None:
        raise SystemExit(__doc__)
    for d in ([cfg_dir] if cfg_dir else []) + [os.path.join(DEFAULT_CONFIG_DIR, "datasets"), DEFAULT_CONFIG_DIR]:
        p = os.path.join(d, name + ".yaml")
        if os.path.isfile(p):
            cfg = yaml.safe_load(open(p, "r", encoding="utf-8")) or {}
            return DataHandlerConfig(apply_overrides(cfg, overrides))
    raise FileNotFoundError(f"dataset config '{name}.yaml' not found")


def _tokenizer(cfg):
    ttype = "HuggingFaceTokenizer" if cfg.tokenizer_type in ("PretrainedFromHF", "HuggingFaceTokenizer") \
        else cfg.tokenizer_type
    return get_tokenizer(cfg.tokenizer_name_or_path, ttype, None, None, use_fast=not cfg.tokenizer_not_use_fast,
                         vocab_size=cfg.pad_vocab_size_to)


def _run_part(payload):
    cfg_dict, rows, part = payload
    cfg = DataHandlerConfig(cfg_dict)
    cfg.output_prefix = f"{cfg.output_prefix}_{part:03d}"
    handler = get_dataset_handler(cfg, rows, _tokenizer(cfg))
    return handler.serialize_to_disk()


def _merge(parts, final_prefixes):
    for field, final in final_prefixes.items():
        first = _Index(get_idx_path(parts[0][field]))
        b = IndexedDatasetBuilder(get_bin_path(final), dtype=first.dtype)
        for p in parts:
            b.add_index(p[field])
        b.finalize(get_idx_path(final))
        for p in parts:
            os.remove(get_bin_path(p[field]))
            os.remove(get_idx_path(p[field]))


def main(argv=None):
    cfg = _load_config(sys.argv[1:] if argv is None else argv)
    validate_data_handler_config(cfg)
    rows = build_dataset(cfg)
    if cfg.n_subs <= 1:
        handler = get_dataset_handler(cfg, rows, _tokenizer(cfg))
        prefixes = handler.serialize_to_disk()
    else:
        chunk = -(-len(rows) // cfg.n_subs)
        base = {k: v for k, v in cfg.dict().items()}
        jobs = [(base, rows[i * chunk:(i + 1) * chunk], i) for i in range(cfg.n_subs) if rows[i * chunk:(i + 1) * chunk]]
        # fresh interpreters: the parent may already run threads (tokenizers, torch), which a fork would copy mid-flight
        with mp.get_context("spawn").Pool(min(cfg.workers, len(jobs))) as pool:
            parts = pool.map(_run_part, jobs)
        prefixes = {f: p.replace("_000_packed", "_packed") for f, p in parts[0].items()}
        _merge(parts, prefixes)
    print("wrote:", {k: v + ".{bin,idx}" for k, v in prefixes.items()})
    return prefixes


if __name__ == "__main__":
    main()
