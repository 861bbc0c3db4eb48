"""Per-prompt store for multimodal inputs next to the text experience store.

Images / videos belong to a *prompt*, not to one of its ``n`` sampled responses, so they are kept
once per prompt and looked up with the sample indexes the text store hands out
(``prompt = index // n_samples_per_prompt``).  A prompt may carry any number of images or videos;
every column is therefore a ragged list per prompt, and a batch is the concatenation of the
requested prompts' items plus the per-prompt counts needed to take it apart again
(``unpack_mm_experience``).

Consumers read fixed column sets (``columns_for``): the rollout reads the raw media (or the
pre-computed vision-encoder embeddings when ``reuse_image_embeds``), the log-prob / update stages
read the processor output (``pixel_values`` + ``image_grid_thw``), the rule reward reads ``labels``.

Reference: ``mindspeed_rl/trainer/utils/mm_transfer_dock.py:14-382`` (``MMGRPOTransferDock``).
"""
from __future__ import annotations

import threading
from typing import Any, Dict, List, Optional, Sequence

import torch

MEDIA_COLUMNS = ("image", "pixel_values", "image_grid_thw", "image_shape", "labels", "vit_embeds", "position_ids",
                 "image_num", "video", "video_shape", "video_fps", "video_num")
_COUNT_COLUMNS = ("image_num", "video_num", "video_fps")
_FLAT_MEDIA = ("image", "video")               # flattened pixels, concatenated along dim 1: [1, sum(numel)]


class MMGRPOTransferDock:
    def __init__(self, prompts_num: int, n_samples_per_prompt: int, reuse_image_embeds: bool = False):
        self.prompts_num = prompts_num
        self.n_samples_per_prompt = n_samples_per_prompt
        self.experience_columns = list(MEDIA_COLUMNS)
        self._lock = threading.Lock()
        self._data: Dict[str, List[Any]] = {c: [None] * prompts_num for c in self.experience_columns}
        processed = ["pixel_values", "image_grid_thw", "image_num", "video_num"]
        self.consumer_columns: Dict[str, List[str]] = {
            "actor_rollout": ["image", "image_shape", "image_num", "video", "video_shape", "video_fps", "video_num"],
            "dynamic_sampling": list(processed),
            "actor_log_prob": list(processed),
            "ref_log_prob": list(processed),
            "actor_train": list(processed),
            "rule_reward": ["labels"],
        }
        if reuse_image_embeds:
            # the vision encoder runs once per prompt (its own stage); everyone else reads its output
            embeds = ["vit_embeds", "image_grid_thw", "image_num", "video_num"]
            self.consumer_columns["actor_image_embeds"] = list(processed)
            for stage in ("actor_rollout", "actor_log_prob", "ref_log_prob", "actor_train"):
                self.consumer_columns[stage] = list(embeds)

    # ---- column sets ------------------------------------------------------------------------------
    def get_columns(self, consumer: str) -> List[str]:
        """Columns ``consumer`` reads, or ``[]`` when it reads none or one of them was never filled
        (a text-only run)."""
        cols = self.consumer_columns.get(consumer, [])
        with self._lock:
            for c in cols:
                if all(v is None for v in self._data[c]):
                    return []
        return list(cols)

    # ---- rows --------------------------------------------------------------------------------------
    def _prompt_rows(self, indexes: Sequence[int], get_n_samples: bool) -> List[int]:
        idx = list(indexes)
        if get_n_samples:
            idx = idx[::self.n_samples_per_prompt]
        return [i // self.n_samples_per_prompt for i in idx]

    def put_experience(self, batch: Dict[str, Sequence[Any]], indexes: Sequence[int]) -> None:
        """``batch[column][i]`` belongs to prompt ``indexes[i]`` (prompt indexes, not sample indexes)."""
        with self._lock:
            for col, items in batch.items():
                if col not in self._data:
                    continue
                for i, item in enumerate(items):
                    self._data[col][indexes[i]] = item

    def get_experience_dict(self, experience_columns: Sequence[str], indexes: Optional[Sequence[int]] = None,
                            get_n_samples: bool = True) -> Dict[str, List[Any]]:
        """Per-prompt items, unmerged.  ``indexes`` are sample indexes of the text store."""
        if indexes is None:
            return {}
        rows = self._prompt_rows(indexes, get_n_samples)
        with self._lock:
            return {c: [self._data[c][r] for r in rows] for c in experience_columns}

    def get_experience(self, consumer: str, experience_columns: Sequence[str],
                       indexes: Optional[Sequence[int]] = None, get_n_samples: bool = True) -> Dict[str, Any]:
        """Merged batch of the prompts behind ``indexes`` (see :func:`merge_mm_columns`)."""
        if indexes is None:
            return {}
        return merge_mm_columns(self.get_experience_dict(experience_columns, indexes, get_n_samples))

    def clear(self) -> None:
        with self._lock:
            for c in self._data:
                self._data[c] = [None] * self.prompts_num


def merge_mm_columns(per_prompt: Dict[str, List[Any]]) -> Dict[str, Any]:
    """Lists of per-prompt items -> one tensor per column: counts become a ``[P, 1]`` column,
    flattened media are joined along dim 1, everything else along dim 0; labels stay a list."""
    out: Dict[str, Any] = {}
    for col, items in per_prompt.items():
        if col == "labels":
            out[col] = list(items)
        elif col in _COUNT_COLUMNS:
            out[col] = torch.as_tensor([float(x) if col == "video_fps" else int(x) for x in _flatten_scalars(items)]) \
                .reshape(-1, 1)
        elif col in _FLAT_MEDIA:
            out[col] = torch.cat(list(items), dim=1)
        else:
            out[col] = torch.cat(list(items), dim=0)
    return out


def _flatten_scalars(items):
    for x in items:
        if torch.is_tensor(x):
            yield from x.reshape(-1).tolist()
        elif isinstance(x, (list, tuple)):
            yield from x
        else:
            yield x


def _split_by(data: torch.Tensor, counts: Sequence[int]) -> List[torch.Tensor]:
    out, start = [], 0
    for n in counts:
        out.append(data[start:start + n])
        start += n
    return out


def split_sizes(shapes: torch.Tensor, merge_size: int = 1) -> List[int]:
    """Rows (or elements) of every item from its shape row: the product of the entries, divided by
    ``merge_size**2`` for vision-encoder outputs after the spatial merge."""
    return [int(torch.as_tensor(s).prod().item()) // (merge_size * merge_size) for s in shapes]


def unpack_mm_experience(batch: Dict[str, Any], merge_size: int = 1) -> Dict[str, Any]:
    """Take a merged batch apart again: per prompt, the list of its images (``[C, H, W]`` tensors) or
    videos, its ``pixel_values`` / ``vit_embeds`` rows and its ``image_grid_thw`` rows.  A batch holds
    images or videos, not both."""
    out = dict(batch)
    n_img = batch.get("image_num")
    n_vid = batch.get("video_num")
    use_images = n_img is not None and int(torch.as_tensor(n_img).sum()) > 0
    counts_t = n_img if use_images else n_vid
    counts = [int(c) for c in torch.as_tensor(counts_t).reshape(-1).tolist()] if counts_t is not None else None
    media, shape_key = ("image", "image_shape") if use_images else ("video", "video_shape")
    if media in batch and shape_key in batch and counts is not None:
        shapes = torch.as_tensor(batch[shape_key]).reshape(-1, torch.as_tensor(batch[shape_key]).shape[-1])
        flat = batch[media].reshape(-1)
        sizes = split_sizes(shapes)
        items = [chunk.reshape(shapes[i].tolist()) for i, chunk in enumerate(_split_by(flat, sizes))]
        out[media] = _split_by(items, counts)
        if not use_images and "video_fps" in batch:
            out["video_fps"] = _split_by(batch["video_fps"].reshape(-1), counts)
    if "image_grid_thw" in batch and counts is not None:
        grid = batch["image_grid_thw"]
        for key, ms in (("pixel_values", 1), ("vit_embeds", merge_size)):
            if key in batch:
                per_item = _split_by(batch[key], split_sizes(grid, ms))
                out[key] = [torch.cat(group) if group else batch[key][:0] for group in _split_by(per_item, counts)]
        out["image_grid_thw"] = _split_by(grid, counts)
    return out
