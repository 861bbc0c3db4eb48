"""Synthetic prompt source for benchmarks and smoke tests: uniform random token ids of a fixed
(or ranged) length, yielded in the batch format of ``PromptDataLoader``
(``{"prompts": [1-D LongTensor, ...], <extra keys>}``)."""
from __future__ import annotations

from typing import Dict, Iterator, List, Optional, Tuple, Union

import torch


class SyntheticPromptLoader:
    def __init__(self, batch_size: int, prompt_length: Union[int, Tuple[int, int]], vocab_size: int,
                 seed: int = 0, num_batches: Optional[int] = None, low_token: int = 0,
                 with_labels: bool = False):
        self.batch_size, self.vocab_size = batch_size, vocab_size
        self.prompt_length = prompt_length
        self.num_batches = num_batches
        self.low_token = low_token
        self.with_labels = with_labels
        self.gen = torch.Generator().manual_seed(seed)

    def __iter__(self) -> Iterator[Dict[str, List[torch.Tensor]]]:
        i = 0
        while self.num_batches is None or i < self.num_batches:
            yield self.next_batch()
            i += 1

    def __next__(self):
        return self.next_batch()

    def next_batch(self) -> Dict[str, List[torch.Tensor]]:
        prompts = []
        for _ in range(self.batch_size):
            if isinstance(self.prompt_length, int):
                n = self.prompt_length
            else:
                n = int(torch.randint(self.prompt_length[0], self.prompt_length[1] + 1, (1,),
                                      generator=self.gen))
            prompts.append(torch.randint(self.low_token, self.vocab_size, (n,), generator=self.gen,
                                         dtype=torch.int64))
        out = {"prompts": prompts}
        if self.with_labels:
            out["labels"] = [torch.tensor([7], dtype=torch.int64) for _ in prompts]
        return out
