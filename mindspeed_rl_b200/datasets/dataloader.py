"""Samplers and data loaders for prompts and pairwise (DPO) batches.

* ``PromptSampler`` -- sequential batches starting at ``consumed_samples`` (how resume skips
  prompts that were already trained on); ``PretrainingSampler`` -- this DP rank's slice of each
  ``micro_batch * dp`` window.
* ``PromptDataLoader`` yields ``{"prompts": [LongTensor...], <extra keys>: [...]}`` -- the batch
  format the trainers put into the experience store.
* ``MultiModalDataLoader`` / pairwise collator for DPO.

Reference: ``mindspeed_rl/datasets/data_samplers.py:4-92``, ``datasets/dataloader.py:14-135``.
"""
from __future__ import annotations

from typing import Dict, Iterator, List, Optional, Sequence

import numpy as np
import torch
from torch.utils.data import DataLoader, RandomSampler, SequentialSampler


class PromptSampler:
    def __init__(self, total_samples: int, consumed_samples: int, batch_size: int, drop_last: bool = True):
        if total_samples <= 0:
            raise ValueError("no samples to consume")
        if consumed_samples >= total_samples:
            raise ValueError(f"consumed_samples {consumed_samples} >= total_samples {total_samples}")
        self.total_samples, self.consumed_samples = total_samples, consumed_samples
        self.batch_size, self.drop_last = batch_size, drop_last

    def __len__(self) -> int:
        return self.total_samples

    def __iter__(self) -> Iterator[List[int]]:
        batch = []
        for idx in range(self.consumed_samples, self.total_samples):
            batch.append(idx)
            if len(batch) == self.batch_size:
                yield batch
                batch = []
        if batch and not self.drop_last:
            yield batch


class PretrainingSampler:
    def __init__(self, total_samples: int, consumed_samples: int, micro_batch_size: int,
                 data_parallel_rank: int, data_parallel_size: int, drop_last: bool = True):
        if data_parallel_rank >= data_parallel_size:
            raise ValueError("data_parallel_rank must be < data_parallel_size")
        self.total_samples, self.consumed_samples = total_samples, consumed_samples
        self.micro_batch_size = micro_batch_size
        self.rank, self.size, self.drop_last = data_parallel_rank, data_parallel_size, drop_last
        self.window = micro_batch_size * data_parallel_size

    def __len__(self) -> int:
        return self.total_samples

    def __iter__(self) -> Iterator[List[int]]:
        lo = self.rank * self.micro_batch_size
        batch = []
        for idx in range(self.consumed_samples, self.total_samples):
            batch.append(idx)
            if len(batch) == self.window:
                yield batch[lo:lo + self.micro_batch_size]
                batch = []
        if batch and not self.drop_last:
            yield batch[lo:lo + self.micro_batch_size]


def _tensor(x) -> torch.Tensor:
    return x if torch.is_tensor(x) else torch.as_tensor(np.asarray(x))


class PromptDataLoader(DataLoader):
    """Batches of prompts (+ additional keys such as ``labels``) as lists of 1-D tensors."""

    def __init__(self, dataset, global_batch_size: int, num_workers: int = 0, seed: int = 1234,
                 dataset_additional_keys: Optional[Sequence[str]] = None, no_shuffle: bool = False,
                 is_pairwise_dataset: bool = False, tokenizer=None, consumed_samples: int = 0):
        keys = list(dataset_additional_keys or [])

        def collate(rows: List[Dict[str, np.ndarray]]) -> Dict[str, List[torch.Tensor]]:
            out: Dict[str, List[torch.Tensor]] = {"prompts": [_tensor(r["input_ids"]).long() for r in rows]}
            for k in keys:
                out[k] = [_tensor(r[k]).long() for r in rows if k in r]
            return out

        def collate_pairwise(rows):
            pad = getattr(tokenizer, "pad_token_id", None) or 0
            out = {}
            for k in ("input_ids", "attention_mask", "labels"):
                seqs = [_tensor(r[f"chosen_{k}"]).long() for r in rows] + \
                       [_tensor(r[f"rejected_{k}"]).long() for r in rows]
                fill = -100 if k == "labels" else (pad if k == "input_ids" else 0)
                out[k] = torch.nn.utils.rnn.pad_sequence(seqs, batch_first=True, padding_value=fill)
            return out

        if no_shuffle:
            sampler = SequentialSampler(dataset)
        else:
            gen = torch.Generator().manual_seed(seed)
            sampler = RandomSampler(dataset, generator=gen)
        super().__init__(dataset, batch_size=global_batch_size, sampler=sampler, num_workers=num_workers,
                         collate_fn=collate_pairwise if is_pairwise_dataset else collate, drop_last=True,
                         pin_memory=False)
        self.consumed_batches = consumed_samples // max(global_batch_size, 1)

    def __iter__(self):
        it = super().__iter__()
        for _ in range(self.consumed_batches):  # resume: skip what was consumed before the restart
            try:
                next(it)
            except StopIteration:
                it = super().__iter__()
        self.consumed_batches = 0
        return it


class InfiniteLoader:
    """Wrap a re-iterable loader into an endless iterator (epoch after epoch)."""

    def __init__(self, loader):
        self.loader = loader
        self._it = iter(loader)

    def __iter__(self):
        return self

    def __next__(self):
        try:
            return next(self._it)
        except StopIteration:
            self._it = iter(self.loader)
            return next(self._it)
