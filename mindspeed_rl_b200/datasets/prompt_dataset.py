"""Prompt / instruction / pairwise datasets over packed indexed files, shuffle-index cache, and
the train/valid/test split builder.

Behaviour follows the reference (``mindspeed_rl/datasets/prompt_dataset.py:15-183``,
``datasets/utils.py:97-176``, ``datasets/build_dataset.py:26-194``): RL prompts are truncated to
``seq_length`` and carry the extra keys named in ``dataset_additional_keys`` (e.g. ``labels``);
instruction samples that exceed the length are cut turn by turn proportionally between prompt
and answer; pairwise samples share the prompt between ``chosen`` and ``rejected``.
"""
from __future__ import annotations

import os
import time
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .indexed_dataset import get_packed_indexed_dataset

IGNORE_INDEX = -100


class BaseDataset(torch.utils.data.Dataset):
    def __init__(self, dataset, dataset_type: str = "base"):
        self.dataset, self.dataset_type = dataset, dataset_type

    def __len__(self):
        return len(self.dataset)

    def get_type(self) -> str:
        return self.dataset_type


def infer_seqlen(source_len: int, target_len: int, cutoff_len: int) -> Tuple[int, int]:
    """Split a token budget between prompt and answer (short sides keep their full length)."""
    if target_len * 2 < cutoff_len:
        max_target = cutoff_len
    elif source_len * 2 < cutoff_len:
        max_target = cutoff_len - source_len
    else:
        max_target = int(cutoff_len * (target_len / (source_len + target_len)))
    new_target = min(max_target, target_len)
    new_source = min(max(cutoff_len - new_target, 0), source_len)
    return new_source, new_target


def get_prompt_index(labels: np.ndarray, ignored_label: int = IGNORE_INDEX) -> Tuple[List[int], List[int]]:
    """Begin / end offsets of every run of ignored labels (= the prompt part of each turn)."""
    is_prompt = np.asarray(labels) == ignored_label
    edges = np.diff(np.concatenate([[0], is_prompt.astype(np.int8), [0]]))
    return np.where(edges == 1)[0].tolist(), np.where(edges == -1)[0].tolist()


def build_shuffle_index(name: str, data_prefix: str, start_index: int, nb_documents: int,
                        num_samples: Optional[int], seed: int, full_shuffle: bool = False,
                        no_shuffle: bool = False, is_leader: bool = True, barrier=None) -> np.ndarray:
    """Sample order over ``[start, start + nb_documents)`` repeated to cover ``num_samples``;
    cached as ``{prefix}_{name}_indexmap_{n}ns_{seed}s_shuffle_idx.npy`` by the leader rank."""
    num_samples = num_samples or nb_documents
    tag = f"{data_prefix}_{name}_indexmap_{num_samples}ns_{seed}s_{'full' if full_shuffle else 'epoch'}"
    path = tag + "_shuffle_idx.npy"
    if is_leader and not os.path.isfile(path):
        rng = np.random.RandomState(seed)
        epochs = -(-num_samples // max(nb_documents, 1))
        docs = np.arange(start_index, start_index + nb_documents)
        if no_shuffle:
            idx = np.tile(docs, epochs)
        elif full_shuffle:
            idx = np.tile(docs, epochs)
            rng.shuffle(idx)
        else:
            idx = np.concatenate([rng.permutation(docs) for _ in range(epochs)])
        try:
            np.save(path, idx[:max(num_samples, nb_documents)], allow_pickle=True)
        except OSError:
            return idx[:max(num_samples, nb_documents)]
    if barrier is not None:
        barrier()
    for _ in range(600):
        if os.path.isfile(path):
            break
        time.sleep(0.1)
    return np.load(path, allow_pickle=True, mmap_mode="r")


class PromptDataset(BaseDataset):
    def __init__(self, data_prefix: str = "", is_packed_data: bool = True, tokenizer=None,
                 seq_length: int = 128, num_samples: Optional[int] = None, name: str = "",
                 documents: Any = None, seed: int = 42, full_shuffle_instruction_dataset: bool = False,
                 no_shuffle: bool = True, pad_token: int = 0, eos_token: int = 1, extra_param: Any = None,
                 **kwargs):
        if not is_packed_data:
            raise NotImplementedError("only packed (preprocessed) datasets are supported")
        self.args = extra_param
        self.seq_length, self.pad_token, self.eos_token = seq_length, pad_token, eos_token
        self.tokenizer = tokenizer
        self.is_pairwise = bool(getattr(extra_param, "is_pairwise_dataset", False))
        self.additional_keys = list(getattr(extra_param, "dataset_additional_keys", []) or [])
        res = get_packed_indexed_dataset(data_prefix, getattr(extra_param, "max_prompt_length", None),
                                         self.is_pairwise)
        documents = documents if documents is not None else np.arange(len(res))
        self.shuffle_index = build_shuffle_index(
            name, data_prefix, int(documents[0]), len(documents), num_samples, seed,
            full_shuffle_instruction_dataset, no_shuffle, kwargs.get("is_leader", True), kwargs.get("barrier"))
        super().__init__(res, "Prompt_DS_Packed")

    def __len__(self) -> int:
        return len(self.shuffle_index)

    def __getitem__(self, index: int) -> Dict[str, np.ndarray]:
        item = self.dataset[int(self.shuffle_index[index])]
        return self._cut_pairwise(item) if self.is_pairwise else self._cut_instruction(item)

    # ------------------------------------------------------------------------------------------
    def _cut_instruction(self, item: Dict[str, np.ndarray]) -> Dict[str, np.ndarray]:
        dt = np.int64
        if "labels" in item and not self.additional_keys:
            ids, labels = item["input_ids"], item["labels"]
            if len(ids) <= self.seq_length:
                return {"input_ids": ids.astype(dt), "attention_mask": np.ones_like(ids).astype(dt),
                        "labels": labels.astype(dt)}
            begins, ends = get_prompt_index(labels)
            out_ids, out_labels, total = [], [], 0
            for t, (b, e) in enumerate(zip(begins, ends)):
                if total >= self.seq_length:
                    break
                nxt = begins[t + 1] if t + 1 < len(begins) else len(labels)
                src, msk, tgt = ids[b:e], labels[b:e], labels[e:nxt]
                s_len, t_len = infer_seqlen(len(src), len(tgt), self.seq_length - total)
                out_ids += [src[:s_len], tgt[:t_len]]
                out_labels += [msk[:s_len], tgt[:t_len]]
                total += s_len + t_len
            ids = np.concatenate(out_ids) if out_ids else ids[:0]
            labels = np.concatenate(out_labels) if out_labels else labels[:0]
            return {"input_ids": ids.astype(dt), "attention_mask": np.ones_like(ids).astype(dt),
                    "labels": labels.astype(dt)}
        ids = item["input_ids"][:self.seq_length]
        out = {"input_ids": ids.astype(dt), "attention_mask": np.ones_like(ids).astype(dt)}
        for k in self.additional_keys:
            if k in item:
                out[k] = item[k]
        return out

    def _cut_pairwise(self, item: Dict[str, np.ndarray]) -> Dict[str, np.ndarray]:
        dt = np.int64
        p_len = int((item["chosen_labels"] != IGNORE_INDEX).nonzero()[0][0])
        prompt = item["chosen_input_ids"][:p_len]
        chosen, rejected = item["chosen_input_ids"][p_len:], item["rejected_input_ids"][p_len:]
        s_len, t_len = infer_seqlen(len(prompt), max(len(chosen), len(rejected)), self.seq_length)
        prompt, chosen, rejected = prompt[:s_len], chosen[:t_len], rejected[:t_len]
        mask = np.full(s_len, IGNORE_INDEX)
        out = {}
        for name, ans in (("chosen", chosen), ("rejected", rejected)):
            ids = np.append(prompt, ans)
            out[f"{name}_input_ids"] = ids.astype(dt)
            out[f"{name}_attention_mask"] = np.ones_like(ids).astype(dt)
            out[f"{name}_labels"] = np.append(mask, ans).astype(dt)
        return out


def get_train_valid_test_split(splits_string: str, size: int) -> List[int]:
    """``"80,10,10"`` -> cumulative document boundaries ``[0, a, b, size]``."""
    parts = [float(s) for s in str(splits_string).replace("/", ",").split(",") if s != ""]
    parts = (parts + [0.0, 0.0, 0.0])[:3]
    total = sum(parts)
    if total <= 0:
        raise ValueError("split must contain a positive share")
    bounds = [0]
    for p in parts:
        bounds.append(bounds[-1] + int(round(p / total * size)))
    diff = bounds[-1] - size
    return [bounds[0]] + [b - diff for b in bounds[1:]]


def build_train_valid_test_datasets(data_prefix, splits_string: str, seq_length: int,
                                    train_valid_test_num_samples: Sequence[Optional[int]],
                                    dataset_cls=PromptDataset, tokenizer=None, parallel_state=None,
                                    full_shuffle_instruction_dataset: bool = False, no_shuffle: bool = False,
                                    seed: int = 1234, extra_param=None, **kwargs):
    """Returns ``(train, valid, test)`` datasets (``None`` for empty splits)."""
    prefix = data_prefix[0] if isinstance(data_prefix, (list, tuple)) else data_prefix
    probe = get_packed_indexed_dataset(prefix, None, bool(getattr(extra_param, "is_pairwise_dataset", False)))
    bounds = get_train_valid_test_split(splits_string, len(probe))
    out = []
    for i, name in enumerate(("train", "valid", "test")):
        lo, hi = bounds[i], bounds[i + 1]
        if hi <= lo:
            out.append(None)
            continue
        out.append(dataset_cls(data_prefix=prefix, is_packed_data=True, tokenizer=tokenizer,
                               seq_length=seq_length, num_samples=train_valid_test_num_samples[i], name=name,
                               documents=np.arange(lo, hi), seed=seed,
                               full_shuffle_instruction_dataset=full_shuffle_instruction_dataset,
                               no_shuffle=no_shuffle, extra_param=extra_param, **kwargs))
    return tuple(out)
