"""Raw dataset -> tokenised ``.bin/.idx`` files (the work of ``cli/preprocess_data.py``).

Pipeline: load json / jsonl / parquet rows -> *align* each row to the intermediate form
``{prompt: [{role, content}...], response: [...], system: [s], tools: [t], <extra keys>}`` (column
names configurable through ``map_keys``) -> a *handler* tokenises it with a chat template ->
fields are streamed into ``{output_prefix}_packed_{field}_document.{bin,idx}``.

Handlers (names as used in the dataset YAMLs; reference: ``mindspeed_rl/datasets/data_handler.py``):
``AlpacaStyleInstructionHandler`` (SFT: input_ids / attention_mask / labels with prompt masked),
``AlpacaStylePairwiseHandler`` (DPO: chosen_* / rejected_*), ``AlpacaStyleProcessRewardHandler``
(PRM: step placeholder token labelled + / -), ``R1AlpacaStyleInstructionHandler`` and
``Math17kAlpacaStyleInstructionHandler`` (RL prompts: prompt ids + ``labels`` = tokenised answer).
"""
from __future__ import annotations

import glob
import json
import os
from typing import Any, Dict, Iterable, Iterator, List, Optional, Sequence

import numpy as np

from .indexed_dataset import IndexedDatasetBuilder, get_bin_path, get_idx_path, optimal_dtype
from .templates import get_model_template

IGNORE = -100


# ----------------------------------------------------------------------------------------------
# loading + alignment
# ----------------------------------------------------------------------------------------------
def load_raw_dataset(path: str) -> List[Dict[str, Any]]:
    """Rows of a ``.json`` / ``.jsonl`` / ``.parquet`` file, or of every such file in a directory."""
    files = [path] if os.path.isfile(path) else sorted(
        f for ext in ("json", "jsonl", "parquet") for f in glob.glob(os.path.join(path, f"*.{ext}")))
    if not files:
        raise FileNotFoundError(f"no json/jsonl/parquet data found at {path}")
    rows: List[Dict[str, Any]] = []
    for f in files:
        if f.endswith(".parquet"):
            import pandas as pd

            rows.extend(pd.read_parquet(f).to_dict(orient="records"))
        elif f.endswith(".jsonl"):
            with open(f, "r", encoding="utf-8") as fh:
                rows.extend(json.loads(line) for line in fh if line.strip())
        else:
            with open(f, "r", encoding="utf-8") as fh:
                data = json.load(fh)
            rows.extend(data if isinstance(data, list) else [data])
    return rows


_DEFAULT_KEYS = dict(prompt="instruction", query="input", response="output", history="history",
                     system="system", chosen="chosen", rejected="rejected")


def _plain(v):
    """numpy containers from parquet -> python."""
    if isinstance(v, np.ndarray):
        return [_plain(x) for x in v.tolist()]
    return v


def align_sample(sample: Dict[str, Any], map_keys: Optional[Dict[str, str]] = None, ranking: bool = False,
                 additional_keys: Sequence[str] = ()) -> Optional[Dict[str, Any]]:
    """Alpaca / Math-17k style row -> intermediate form; ``None`` when prompt or answer is empty."""
    keys = dict(_DEFAULT_KEYS)
    keys.update(map_keys or {})
    prompt: List[Dict[str, str]] = []
    for turn in _plain(sample.get(keys["history"])) or []:
        if isinstance(turn, (list, tuple)) and len(turn) == 2:
            prompt += [{"role": "user", "content": turn[0]}, {"role": "assistant", "content": turn[1]}]
    p = _plain(sample.get(keys["prompt"]))
    if isinstance(p, list):        # chat-style prompt: [{"role": "user", "content": ...}]
        parts = [m.get("content", "") for m in p if isinstance(m, dict)]
    else:
        parts = [p] if p else []
    q = sample.get(keys["query"])
    if q:
        parts.append(q)
    text = "\n".join(str(x) for x in parts if x)
    if not text:
        return None
    prompt.append({"role": "user", "content": text})
    if ranking:
        ch, rj = _plain(sample.get(keys["chosen"])), _plain(sample.get(keys["rejected"]))
        if isinstance(ch, list) and ch and rj is None:   # "output": [chosen, rejected]
            ch, rj = ch[0], ch[1] if len(ch) > 1 else None
        if not ch or not rj:
            return None
        response = [{"role": "assistant", "content": str(ch)}, {"role": "assistant", "content": str(rj)}]
    else:
        r = _plain(sample.get(keys["response"]))
        if isinstance(r, dict):     # {"ground_truth": ...} (math-17k reward_model column)
            r = r.get("ground_truth")
        if r is None or r == "":
            return None
        response = [{"role": "assistant", "content": str(r)}]
    out = {"prompt": prompt, "response": response, "system": [sample.get(keys["system"]) or ""], "tools": [""]}
    for k in additional_keys:
        if k != "labels" and k in sample:
            out[k] = sample[k]
    return out


# ----------------------------------------------------------------------------------------------
# handlers
# ----------------------------------------------------------------------------------------------
class BaseDatasetHandler:
    fields: List[str] = ["input_ids"]
    ranking = False

    def __init__(self, args, raw_datasets: Iterable[Dict[str, Any]], tokenizer, splitter=None):
        self.args, self.raw, self.tokenizer, self.splitter = args, raw_datasets, tokenizer, splitter
        self.hf = getattr(tokenizer, "tokenizer", tokenizer)
        self.template = None
        if getattr(args, "prompt_type", None):
            self.template = get_model_template(args.prompt_type.strip(), args.prompt_type_path.strip(),
                                               getattr(args, "enable_thinking", False))
        self.additional_keys = list(getattr(args, "dataset_additional_keys", []) or [])
        self.output_prefix = args.output_prefix + "_packed"

    def tokenize(self, example: Dict[str, Any]) -> Optional[Dict[str, List[int]]]:
        raise NotImplementedError

    def _messages(self, ex):
        if len(ex["prompt"]) % 2 != 1 or len(ex["response"]) < 1:
            return [{"role": "user", "content": ""}, {"role": "assistant", "content": ""}]
        return ex["prompt"] + ex["response"][:1]

    def get_tokenized_data(self) -> Iterator[Dict[str, List[int]]]:
        for row in self.raw:
            ex = align_sample(row, getattr(self.args, "map_keys", None), self.ranking, self.additional_keys)
            if ex is None:
                continue
            tok = self.tokenize(ex)
            if tok is not None:
                yield tok

    def serialize_to_disk(self, iteration_batch_size: int = 50) -> Dict[str, str]:
        """Write one ``.bin/.idx`` pair per field; returns ``{field: path prefix}``."""
        vocab = getattr(self.hf, "vocab_size", None) or len(self.hf)
        builders: Dict[str, IndexedDatasetBuilder] = {}
        prefixes: Dict[str, str] = {}
        count = 0
        for tok in self.get_tokenized_data():
            for f, ids in tok.items():
                if f not in builders:
                    prefixes[f] = f"{self.output_prefix}_{f}_document"
                    dtype = np.int32 if (f.endswith("labels") or min(ids, default=0) < 0) else optimal_dtype(vocab)
                    builders[f] = IndexedDatasetBuilder(get_bin_path(prefixes[f]), dtype=dtype)
                builders[f].add_item(np.asarray(ids))
                builders[f].end_document()
            count += 1
            if count % max(getattr(self.args, "log_interval", 1000), 1) == 0:
                print(f"[preprocess] {count} samples")
        for f, b in builders.items():
            b.finalize(get_idx_path(prefixes[f]))
        return prefixes


class AlpacaStyleInstructionHandler(BaseDatasetHandler):
    fields = ["input_ids", "attention_mask", "labels"]
    train_on_inputs = False

    def tokenize(self, ex):
        ids: List[int] = []
        labels: List[int] = []
        tpl = self.template
        for src, tgt in tpl.encode_multiturn(self.hf, self._messages(ex), ex["system"][0], ex["tools"][0]):
            if self.train_on_inputs:
                mask = src
            elif ids and tpl.efficient_eos:
                mask = [self.hf.eos_token_id] + [IGNORE] * (len(src) - 1)
            else:
                mask = [IGNORE] * len(src)
            ids += src + tgt
            labels += mask + tgt
        if tpl.efficient_eos:
            ids.append(self.hf.eos_token_id)
            labels.append(self.hf.eos_token_id)
        if getattr(self.args, "append_eod", False):
            eod = getattr(self.tokenizer, "eod", self.hf.eos_token_id)
            ids.append(eod)
            labels.append(eod)
        if not ids:
            return None
        return {"input_ids": ids, "attention_mask": [1] * len(ids), "labels": labels}


class AlpacaStylePairwiseHandler(BaseDatasetHandler):
    fields = ["chosen_input_ids", "chosen_labels", "rejected_input_ids", "rejected_labels"]
    ranking = True

    def tokenize(self, ex):
        tpl = self.template
        out = {}
        prompt_msgs = ex["prompt"]
        for name, resp in zip(("chosen", "rejected"), ex["response"]):
            p_ids, a_ids = tpl.encode_oneturn(self.hf, prompt_msgs + [resp], ex["system"][0], ex["tools"][0])
            if tpl.efficient_eos:
                a_ids = a_ids + [self.hf.eos_token_id]
            out[f"{name}_input_ids"] = p_ids + a_ids
            out[f"{name}_labels"] = [IGNORE] * len(p_ids) + a_ids
        return out


class AlpacaStyleProcessRewardHandler(BaseDatasetHandler):
    """Process reward model data: the ``placeholder_token`` that ends each reasoning step is
    labelled with the id of the matching ``reward_tokens`` entry (e.g. ``+`` / ``-``)."""
    fields = ["input_ids", "labels"]

    def tokenize(self, ex):
        text = ex["prompt"][-1]["content"]
        marks = ex["response"][0]["content"]
        ph = self.hf.encode(self.args.placeholder_token, add_special_tokens=False)[-1]
        ids = self.hf.encode(text, add_special_tokens=False)
        try:
            step_labels = json.loads(marks) if marks.strip().startswith("[") else marks.split()
        except json.JSONDecodeError:
            step_labels = marks.split()
        reward_ids = [self.hf.encode(str(s), add_special_tokens=False)[-1] for s in step_labels]
        labels = [IGNORE] * len(ids)
        pos = [i for i, t in enumerate(ids) if t == ph]
        if len(pos) != len(reward_ids):
            return None
        for i, r in zip(pos, reward_ids):
            labels[i] = r
        return {"input_ids": ids, "labels": labels}


class R1AlpacaStyleInstructionHandler(BaseDatasetHandler):
    """RL prompts: ``input_ids`` = rendered prompt, ``labels`` = tokenised reference answer."""

    def __init__(self, args, raw_datasets, tokenizer, splitter=None):
        super().__init__(args, raw_datasets, tokenizer, splitter)
        self.fields = ["input_ids", "attention_mask", *self.additional_keys]

    def tokenize(self, ex):
        ids: List[int] = []
        for src, _ in self.template.encode_multiturn(self.hf, self._messages(ex), ex["system"][0], ex["tools"][0]):
            ids += src
        if not ids:
            return None
        out = {"input_ids": ids, "attention_mask": [1] * len(ids)}
        for k in self.additional_keys:
            text = ex["response"][-1]["content"] if k == "labels" else str(ex.get(k, ""))
            out[k] = self.hf.encode(text, padding=False, add_special_tokens=False)
        return out


class Math17kAlpacaStyleInstructionHandler(R1AlpacaStyleInstructionHandler):
    """Same tokenisation; rows use the math-17k columns (``prompt`` chat list, ``reward_model``)."""


_HANDLERS = {c.__name__: c for c in (AlpacaStyleInstructionHandler, AlpacaStylePairwiseHandler,
                                     AlpacaStyleProcessRewardHandler, R1AlpacaStyleInstructionHandler,
                                     Math17kAlpacaStyleInstructionHandler)}


def get_dataset_handler(args, raw_dataset, tokenizer, splitter=None) -> BaseDatasetHandler:
    name = args.handler_name
    if name not in _HANDLERS:
        raise ValueError(f"unknown handler '{name}' (available: {sorted(_HANDLERS)})")
    return _HANDLERS[name](args, raw_dataset, tokenizer, splitter)


def build_dataset(args) -> List[Dict[str, Any]]:
    return load_raw_dataset(args.input)
