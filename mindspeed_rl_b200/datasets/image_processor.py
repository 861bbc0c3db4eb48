"""Image pre-processing for vision-language prompts (Qwen2-VL family layout).

An image becomes ``pixel_values [grid_h * grid_w, C * T * P * P]`` (one row per ``P x P`` patch,
``T`` = 2 temporal copies of a still image) plus its ``image_grid_thw = (1, grid_h, grid_w)``.  Rows
are ordered so that the ``merge x merge`` patches that the vision tower later merges into one token
are neighbours.  The language-model prompt gets ``grid_h * grid_w / merge^2`` placeholder tokens per
image.  Behaviour follows the processor the reference calls
(``mindspeed_rl/datasets/multimodal_dataset.py:63-96``: ``processor.image_processor`` with
``merge_size``, ``min_pixels`` / ``max_pixels`` limits as in ``mm_utils.process_image``).
"""
from __future__ import annotations

import math
from typing import List, Sequence, Tuple, Union

import numpy as np
import torch

MEAN = (0.48145466, 0.4578275, 0.40821073)
STD = (0.26862954, 0.26130258, 0.27577711)


def smart_resize(h: int, w: int, factor: int, min_pixels: int, max_pixels: int) -> Tuple[int, int]:
    """Height / width rounded to multiples of ``factor`` with the pixel count kept inside the limits
    and the aspect ratio kept as far as the rounding allows."""
    hb = max(factor, round(h / factor) * factor)
    wb = max(factor, round(w / factor) * factor)
    if hb * wb > max_pixels:
        beta = math.sqrt(h * w / max_pixels)
        hb = max(factor, math.floor(h / beta / factor) * factor)
        wb = max(factor, math.floor(w / beta / factor) * factor)
    elif hb * wb < min_pixels:
        beta = math.sqrt(min_pixels / (h * w))
        hb = math.ceil(h * beta / factor) * factor
        wb = math.ceil(w * beta / factor) * factor
    return hb, wb


def to_chw_float(image) -> torch.Tensor:
    """PIL image, file path, ``[H, W, 3]`` uint8 array or ``[3, H, W]`` tensor -> float ``[3, H, W]`` in [0, 1]."""
    if isinstance(image, str):
        from PIL import Image

        image = Image.open(image)
    if hasattr(image, "convert"):                      # PIL
        image = np.asarray(image.convert("RGB"))
    t = torch.as_tensor(np.asarray(image)) if not torch.is_tensor(image) else image
    if t.dim() == 3 and t.shape[-1] == 3 and t.shape[0] != 3:
        t = t.permute(2, 0, 1)
    t = t.float()
    return t / 255.0 if t.max() > 1.5 else t


class ImageProcessor:
    def __init__(self, patch_size: int = 14, merge_size: int = 2, temporal_patch_size: int = 2,
                 min_pixels: int = 56 * 56, max_pixels: int = 2048 * 2048):
        self.patch_size, self.merge_size, self.temporal_patch_size = patch_size, merge_size, temporal_patch_size
        self.min_pixels, self.max_pixels = min_pixels, max_pixels

    def tokens_for(self, grid_thw: Sequence[int]) -> int:
        t, h, w = (int(x) for x in grid_thw)
        return t * h * w // (self.merge_size ** 2)

    def __call__(self, images: Sequence[Union[str, np.ndarray, torch.Tensor]]):
        """Returns ``dict(pixel_values [sum patches, C*T*P*P], image_grid_thw [n, 3])``."""
        p, m, tp = self.patch_size, self.merge_size, self.temporal_patch_size
        rows, grids = [], []
        mean, std = torch.tensor(MEAN).view(3, 1, 1), torch.tensor(STD).view(3, 1, 1)
        for img in images:
            x = to_chw_float(img)
            h, w = smart_resize(x.shape[1], x.shape[2], p * m, self.min_pixels, self.max_pixels)
            x = torch.nn.functional.interpolate(x.unsqueeze(0), size=(h, w), mode="bilinear", align_corners=False,
                                                antialias=True)[0]
            x = (x - mean) / std
            gh, gw = h // p, w // p
            frames = x.unsqueeze(0).expand(tp, -1, -1, -1)                            # [T, C, H, W]
            # [T, C, gh/m, m, P, gw/m, m, P] -> rows in (gh/m, gw/m, m, m) order, columns (C, T, P, P)
            v = frames.reshape(tp, 3, gh // m, m, p, gw // m, m, p).permute(2, 5, 3, 6, 1, 0, 4, 7)
            rows.append(v.reshape(gh * gw, 3 * tp * p * p).contiguous())
            grids.append([1, gh, gw])
        return dict(pixel_values=torch.cat(rows) if rows else torch.zeros(0, 3 * tp * p * p),
                    image_grid_thw=torch.tensor(grids, dtype=torch.int64).reshape(-1, 3))
