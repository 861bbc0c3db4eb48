"""Vision-language prompt dataset.

Rows come from JSON-lines or parquet files with a prompt (chat messages or a string containing
``<image>`` markers), the images (paths, nested arrays or tensors) and the reference answer.  Every
``<image>`` marker is expanded to ``<|vision_start|>`` + one placeholder token per merged vision
patch + ``<|vision_end|>``; the row then carries what the multimodal experience store keeps per
prompt: ``pixel_values``, ``image_grid_thw``, ``image_num``, the flattened raw ``image`` with its
``image_shape``, the three-axis rotary ``position_ids`` and ``labels``
(reference: ``mindspeed_rl/datasets/multimodal_dataset.py:17-206``).
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Iterator, List, Optional, Sequence

import torch

from .image_processor import ImageProcessor, to_chw_float
from .mm_utils import get_rope_index

IMAGE_MARK = "<image>"


def load_rows(path: str) -> List[Dict[str, Any]]:
    files = sorted(os.path.join(path, f) for f in os.listdir(path)) if os.path.isdir(path) else [path]
    rows: List[Dict[str, Any]] = []
    for f in files:
        if f.endswith(".parquet"):
            import pyarrow.parquet as pq

            rows.extend(pq.read_table(f).to_pylist())
        elif f.endswith((".jsonl", ".json")):
            with open(f) as fh:
                text = fh.read().strip()
            rows.extend(json.loads(text) if text.startswith("[") else [json.loads(l) for l in text.splitlines() if l])
    return rows


class MultiModalDataset(torch.utils.data.Dataset):
    def __init__(self, data_path_or_rows, tokenizer, processor: Optional[ImageProcessor] = None,
                 prompt_key: str = "prompt", image_key: str = "images", answer_key: str = "answer",
                 max_prompt_length: int = 1024, image_token_id: int = 151655, vision_start_token_id: int = 151652,
                 vision_end_token_id: int = 151653, truncation: str = "error"):
        self.rows = load_rows(data_path_or_rows) if isinstance(data_path_or_rows, str) else list(data_path_or_rows)
        self.tokenizer, self.processor = tokenizer, processor or ImageProcessor()
        self.prompt_key, self.image_key, self.answer_key = prompt_key, image_key, answer_key
        self.max_prompt_length, self.truncation = max_prompt_length, truncation
        self.image_token_id = image_token_id
        self.vision_start_token_id, self.vision_end_token_id = vision_start_token_id, vision_end_token_id

    def __len__(self) -> int:
        return len(self.rows)

    def _text(self, prompt) -> str:
        if isinstance(prompt, str):
            return prompt
        parts = []
        for msg in prompt:                                   # chat messages
            content = msg["content"]
            if isinstance(content, list):
                content = "".join(IMAGE_MARK if c.get("type") == "image" else c.get("text", "") for c in content)
            parts.append(f"{msg.get('role', 'user')}: {content}\n")
        return "".join(parts) + "assistant: "

    def _encode(self, text: str) -> List[int]:
        tok = self.tokenizer
        if hasattr(tok, "tokenize"):
            return list(tok.tokenize(text))
        return list(tok.encode(text, add_special_tokens=False))

    def __getitem__(self, index: int) -> Dict[str, Any]:
        row = dict(self.rows[index])
        images = list(row.get(self.image_key) or [])
        text = self._text(row[self.prompt_key])
        pieces = text.split(IMAGE_MARK)
        if len(pieces) - 1 != len(images):
            raise ValueError(f"row {index}: {len(pieces) - 1} image markers but {len(images)} images")
        mm = self.processor(images)
        ids: List[int] = []
        for i, piece in enumerate(pieces):
            if piece:
                ids.extend(self._encode(piece))
            if i < len(images):
                n = self.processor.tokens_for(mm["image_grid_thw"][i].tolist())
                ids.extend([self.vision_start_token_id] + [self.image_token_id] * n + [self.vision_end_token_id])
        if len(ids) > self.max_prompt_length:
            if self.truncation == "error":
                raise ValueError(f"row {index}: prompt of {len(ids)} tokens exceeds max_prompt_length "
                                 f"{self.max_prompt_length}")
            ids = ids[-self.max_prompt_length:] if self.truncation == "left" else ids[:self.max_prompt_length]
        input_ids = torch.tensor(ids, dtype=torch.int64)
        pos, _ = get_rope_index(input_ids.unsqueeze(0), mm["image_grid_thw"] if images else None,
                                spatial_merge_size=self.processor.merge_size, image_token_id=self.image_token_id,
                                vision_start_token_id=self.vision_start_token_id)
        raw = [to_chw_float(im) for im in images]
        out = dict(prompts=input_ids, input_ids=input_ids, prompt_length=torch.tensor([len(ids)]),
                   position_ids=pos[:, 0].t().contiguous(),          # [S, 3]: rows of the store are concatenated on dim 0
                   labels=row.get(self.answer_key, ""), image_num=len(images), video_num=0,
                   pixel_values=mm["pixel_values"], image_grid_thw=mm["image_grid_thw"])
        if raw:
            out["image"] = torch.cat([r.reshape(1, -1) for r in raw], dim=1)
            out["image_shape"] = torch.tensor([list(r.shape) for r in raw])
        return out


class MultiModalPromptLoader:
    """Batches of ``global_batch_size`` rows in the two-part form the trainers consume: text columns
    for the experience store, media columns (keyed by prompt) for the multimodal store."""

    TEXT = ("prompts", "prompt_length")
    MEDIA = ("pixel_values", "image_grid_thw", "image_num", "video_num", "image", "image_shape", "labels",
             "position_ids")

    def __init__(self, dataset: MultiModalDataset, global_batch_size: int, seed: int = 0, shuffle: bool = True):
        self.dataset, self.gbs, self.seed, self.shuffle = dataset, global_batch_size, seed, shuffle

    def __iter__(self) -> Iterator[Dict[str, Any]]:
        g = torch.Generator().manual_seed(self.seed)
        epoch = 0
        while True:
            order = torch.randperm(len(self.dataset), generator=g).tolist() if self.shuffle else list(range(len(self.dataset)))
            for s in range(0, len(order) - self.gbs + 1, self.gbs):
                rows = [self.dataset[i] for i in order[s:s + self.gbs]]
                batch: Dict[str, Any] = {k: [r[k] for r in rows] for k in self.TEXT}
                batch["mm"] = {k: [r.get(k) for r in rows] for k in self.MEDIA if any(k in r for r in rows)}
                yield batch
            epoch += 1
