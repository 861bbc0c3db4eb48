"""Ragged <-> padded conversions used on the wire between the experience store and workers.

Wire format (reference: ``mindspeed_rl/utils/pad_process.py:12-40``): a dict of padded 2-D
tensors, one per column, plus ``original_length`` -- a 1-D tensor holding the true length of
every row, column after column in dict order.  Plain ``dict`` replaces ``TensorDict``.

All helpers are vectorised (one gather / scatter per call); nothing calls ``.item()`` per row.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Union

import torch
import torch.nn.functional as F

RaggedColumn = Union[torch.Tensor, Sequence[torch.Tensor]]


def pad_rows(rows: Sequence[torch.Tensor], pad_value=0, multiple: int = 1,
             width: Optional[int] = None) -> torch.Tensor:
    """Stack 1-D rows into ``[n, W]`` with ``W`` = max length rounded up to ``multiple``."""
    if len(rows) == 0:
        return torch.empty(0, 0)
    longest = max(int(r.numel()) for r in rows)
    w = width if width is not None else -(-longest // multiple) * multiple
    out = rows[0].new_full((len(rows), w), pad_value)
    for i, r in enumerate(rows):
        n = min(int(r.numel()), w)
        if n:
            out[i, :n] = r.reshape(-1)[:n]
    return out


def pad_multiple(data_list: List[torch.Tensor], pad_id, multiple: int = 1) -> torch.Tensor:
    return pad_rows(data_list, pad_id, multiple)


def padding_dict_to_tensor_dict(experience: Dict[str, RaggedColumn]) -> Dict[str, torch.Tensor]:
    """Ragged columns -> padded columns + ``original_length``."""
    batch: Dict[str, torch.Tensor] = {}
    lengths: List[int] = []
    for name, rows in experience.items():
        rows = list(rows)
        batch[name] = pad_rows(rows, 0)
        lengths.extend(int(r.numel()) for r in rows)
    batch["original_length"] = torch.tensor(lengths, dtype=torch.int64)
    return batch


def truncate_rows(tensor: torch.Tensor, lengths: torch.Tensor, left_pad: bool = False
                  ) -> List[torch.Tensor]:
    """Split a padded ``[n, W]`` tensor into ``n`` CPU rows of the given lengths.

    A row of length 0 whose first element is ``-1`` stands for "no data" and becomes an empty
    int32 tensor (reference: ``pad_process.py:143-166``).
    """
    t = tensor.detach().cpu()
    ls = lengths.detach().cpu().reshape(-1).tolist()
    out = []
    for i, n in enumerate(ls):
        n = int(n)
        if n == 0 and t.size(1) > 0 and t[i, 0].item() == -1:
            out.append(torch.tensor([], dtype=torch.int32))
        elif left_pad:
            out.append(t[i, t.size(1) - n:] if n else t[i, :0])
        else:
            out.append(t[i, :n])
    return out


def remove_padding_tensor_dict_to_dict(data: Optional[Dict[str, torch.Tensor]]
                                       ) -> Dict[str, List[torch.Tensor]]:
    """Inverse of :func:`padding_dict_to_tensor_dict`."""
    if data is None:
        return {}
    if "original_length" not in data:
        return data
    lengths = data["original_length"]
    out: Dict[str, List[torch.Tensor]] = {}
    col = 0
    for name, value in data.items():
        if name == "original_length":
            continue
        n = len(value)
        out[name] = truncate_rows(value, lengths[col * n:(col + 1) * n])
        col += 1
    return out


def remove_padding_and_split_to_list(responses: torch.Tensor, eos_token_id: int,
                                     pad_token_id: int, to_list: bool = False):
    """Cut every row at its first pad token; the EOS is kept when pad == eos."""
    is_pad = responses == pad_token_id
    has_pad = is_pad.any(dim=1)
    first = torch.where(has_pad, is_pad.float().argmax(dim=1),
                        torch.full_like(has_pad, responses.size(1), dtype=torch.int64))
    keep = first + 1 if pad_token_id == eos_token_id else first
    keep = keep.clamp(max=responses.size(1)).tolist()
    rows = []
    for i, n in enumerate(keep):
        row = responses[i, :n]
        rows.append(row[:-1].cpu().tolist() if to_list else row)
    return rows


def _window_gather(src: torch.Tensor, start: torch.Tensor, stop: torch.Tensor, width: int,
                   pad_value) -> torch.Tensor:
    """out[b, j] = src[b, start[b]+j] for j < stop[b]-start[b], else pad."""
    seq = src.size(1)
    start = start.clamp(0, seq).to(torch.int64)
    stop = stop.clamp(0, seq).to(torch.int64)
    j = torch.arange(width, device=src.device).unsqueeze(0)
    idx = start.unsqueeze(1) + j
    valid = idx < stop.unsqueeze(1)
    idx = idx.clamp(max=max(seq - 1, 0))
    if src.dim() == 3:
        g = src.gather(1, idx.unsqueeze(-1).expand(-1, -1, src.size(2)))
        return torch.where(valid.unsqueeze(-1), g, torch.full_like(g, pad_value))
    g = src.gather(1, idx)
    return torch.where(valid, g, torch.full_like(g, pad_value))


def truncate_middle_and_pad(responses: torch.Tensor, input_tensor: torch.Tensor,
                            truncate_lengths: torch.Tensor, pad_value=0.0) -> torch.Tensor:
    """Keep ``input[b, s:e]`` (3-D input) left-aligned in a ``responses.shape[-1]`` wide tensor."""
    return _window_gather(input_tensor, truncate_lengths[:, 0], truncate_lengths[:, 1],
                          responses.shape[-1], pad_value)


def truncate_prompt_and_pad(responses: torch.Tensor, input_tensor: torch.Tensor,
                            truncate_lengths: torch.Tensor, pad_value=0.0) -> torch.Tensor:
    """2-D variant of :func:`truncate_middle_and_pad`."""
    return _window_gather(input_tensor, truncate_lengths[:, 0], truncate_lengths[:, 1],
                          responses.shape[-1], pad_value)


def response_window(prompt_length: torch.Tensor, response_length: torch.Tensor) -> torch.Tensor:
    """``[B, 2]`` (start, stop) of the positions whose next-token prediction is a response token:
    ``[prompt_len - 1, prompt_len + resp_len - 1)`` (reference: ``base_loss_func.py:49-53``)."""
    p = prompt_length.reshape(-1).to(torch.int64)
    r = response_length.reshape(-1).to(torch.int64)
    return torch.stack([p - 1, p + r - 1], dim=1)
