"""Multimodal position helpers.

``get_rope_index`` builds the three-axis (temporal, height, width) rotary position ids of the
Qwen2-VL family: text tokens advance all three axes together; the placeholder tokens of an image or
video of grid ``(t, h, w)`` (after the ``spatial_merge_size`` x ``spatial_merge_size`` patch merge)
get ``(t_idx, h_idx, w_idx)`` offsets from the position where the vision block starts; the text
after a vision block continues from the largest position used so far plus one.  Returns the ids
``[3, batch, seq]`` and, per sequence, the difference between the next position and the sequence
length (what decoding adds to its step counter).

Reference: ``mindspeed_rl/datasets/mm_utils.py:18-239`` (``get_rope_index`` for Qwen2-VL / Qwen2.5-VL).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch


def get_rope_index(input_ids: torch.Tensor, image_grid_thw: Optional[torch.Tensor] = None,
                   video_grid_thw: Optional[torch.Tensor] = None, attention_mask: Optional[torch.Tensor] = None,
                   spatial_merge_size: int = 2, image_token_id: int = 151655, video_token_id: int = 151656,
                   vision_start_token_id: int = 151652, second_per_grid_ts: Optional[torch.Tensor] = None,
                   tokens_per_second: float = 0.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """``input_ids [B, S]`` -> ``(position_ids [3, B, S], deltas [B, 1])``.  Padded positions
    (``attention_mask == 0``) get 1.  ``second_per_grid_ts`` with ``tokens_per_second`` > 0 scales the
    temporal axis of videos (Qwen2.5-VL); otherwise the temporal index is the frame-group index."""
    b, s = input_ids.shape
    if attention_mask is None:
        attention_mask = torch.ones_like(input_ids)
    has_vision = (image_grid_thw is not None and len(image_grid_thw)) or \
        (video_grid_thw is not None and len(video_grid_thw))
    if not has_vision:
        pos = attention_mask.long().cumsum(-1) - 1
        pos = pos.masked_fill(attention_mask == 0, 1)
        deltas = (pos.max(-1, keepdim=True).values + 1 - s).to(input_ids.dtype)
        return pos.unsqueeze(0).expand(3, -1, -1).clone(), deltas
    out = torch.ones(3, b, s, dtype=torch.long, device=input_ids.device)
    deltas = []
    img_i = vid_i = 0
    for row in range(b):
        keep = attention_mask[row] == 1
        ids = input_ids[row][keep].tolist()
        parts = []                                  # [3, n] pieces
        nxt = 0                                     # next free position
        i = 0
        while i < len(ids):
            tok = ids[i]
            if tok in (image_token_id, video_token_id):
                if tok == image_token_id:
                    t, h, w = (int(x) for x in image_grid_thw[img_i])
                    img_i += 1
                    scale = 1.0
                else:
                    t, h, w = (int(x) for x in video_grid_thw[vid_i])
                    scale = 1.0
                    if second_per_grid_ts is not None and tokens_per_second > 0:
                        scale = float(second_per_grid_ts[vid_i]) * tokens_per_second
                    vid_i += 1
                gh, gw = h // spatial_merge_size, w // spatial_merge_size
                n = t * gh * gw
                if ids[i:i + n] != [tok] * n:
                    raise ValueError(f"sequence {row}: expected {n} placeholder tokens for a {t}x{h}x{w} grid")
                ti = (torch.arange(t).view(-1, 1).expand(-1, gh * gw).flatten().float() * scale).long()
                hi = torch.arange(gh).view(1, -1, 1).expand(t, -1, gw).flatten()
                wi = torch.arange(gw).view(1, 1, -1).expand(t, gh, -1).flatten()
                block = torch.stack([ti, hi, wi]) + nxt
                parts.append(block)
                nxt = int(block.max()) + 1
                i += n
            else:
                j = i
                while j < len(ids) and ids[j] not in (image_token_id, video_token_id):
                    j += 1
                parts.append((torch.arange(j - i) + nxt).view(1, -1).expand(3, -1))
                nxt += j - i
                i = j
        pos = torch.cat(parts, dim=1) if parts else torch.zeros(3, 0, dtype=torch.long)
        out[:, row, keep] = pos.to(out.device)
        deltas.append(nxt - s)
    return out, torch.tensor(deltas, device=input_ids.device).view(-1, 1)


def mrope_table(position_ids: torch.Tensor, base_table: torch.Tensor, sections=(16, 24, 24)) -> torch.Tensor:
    """Per-token rotary table for three-axis positions.  ``position_ids [T, 3]`` (temporal, height,
    width), ``base_table [max_pos, d] = [cos | sin]`` of the one-axis rotary embedding, ``sections``:
    how many of the ``d / 2`` frequencies follow each axis (scaled when ``d / 2`` differs from their
    sum).  Returns ``[T, d]``: token ``t`` uses row ``t`` (rotate-half pairing, as ``ops.rope_`` expects)."""
    half = base_table.shape[1] // 2
    total = sum(sections)
    bounds, acc = [0], 0
    for sct in sections:
        acc += sct
        bounds.append(round(acc * half / total))
    pos = position_ids.long().clamp(0, base_table.shape[0] - 1)
    out = torch.empty(pos.shape[0], 2 * half, dtype=base_table.dtype, device=base_table.device)
    for axis in range(3):
        lo, hi = bounds[axis], bounds[axis + 1]
        rows = base_table[pos[:, axis].to(base_table.device)]
        out[:, lo:hi] = rows[:, lo:hi]
        out[:, half + lo:half + hi] = rows[:, half + lo:half + hi]
    return out


def extend_positions(prompt_pos: torch.Tensor, n_new: int) -> torch.Tensor:
    """Three-axis positions of a prompt ``[P, 3]`` followed by ``n_new`` text tokens: generated tokens
    advance all axes together from the largest position of the prompt."""
    if prompt_pos.numel() == 0:
        start = 0
    else:
        start = int(prompt_pos.max()) + 1
    tail = torch.arange(start, start + n_new, dtype=prompt_pos.dtype).unsqueeze(-1).expand(n_new, 3)
    return torch.cat([prompt_pos, tail], dim=0)
