"""Masked reductions shared by losses, advantages and metrics.

Semantics follow ``mindspeed_rl/utils/torch_functional.py:22-105``: the masked mean uses
``sum(x*m) / (sum(m) + 1e-8)``; the masked variance is Bessel-corrected by default and
refuses a mask that selects no element (or one element when unbiased).
"""
from __future__ import annotations

from typing import Optional

import torch

_EPS = 1e-8


def masked_sum(values: torch.Tensor, mask: torch.Tensor, axis: Optional[int] = None) -> torch.Tensor:
    prod = values * mask
    return prod.sum() if axis is None else prod.sum(dim=axis)


def masked_mean(values: torch.Tensor, mask: torch.Tensor, axis: Optional[int] = None) -> torch.Tensor:
    if axis is None:
        return (values * mask).sum() / (mask.sum() + _EPS)
    return (values * mask).sum(dim=axis) / (mask.sum(dim=axis) + _EPS)


def masked_var(values: torch.Tensor, mask: torch.Tensor, unbiased: bool = True) -> torch.Tensor:
    mean = masked_mean(values, mask)
    var = masked_mean((values - mean) ** 2, mask)
    if unbiased:
        count = mask.sum()
        if count == 0:
            raise ValueError("masked_var: the mask selects no element")
        if count == 1:
            raise ValueError("masked_var: an unbiased variance needs at least two elements")
        var = var * (count / (count - 1))
    return var


def masked_whiten(values: torch.Tensor, mask: torch.Tensor, shift_mean: bool = True) -> torch.Tensor:
    mean, var = masked_mean(values, mask), masked_var(values, mask)
    out = (values - mean) * torch.rsqrt(var + _EPS)
    if not shift_mean:
        out = out + mean
    return out


def clip_by_value(x: torch.Tensor, lo: torch.Tensor, hi: torch.Tensor) -> torch.Tensor:
    """Element-wise clamp with tensor bounds."""
    return torch.maximum(torch.minimum(x, hi), lo)


def sequence_mask(lengths: torch.Tensor, width: int, dtype=torch.float32) -> torch.Tensor:
    """``[B, width]`` mask with ones in the first ``lengths[b]`` columns."""
    ar = torch.arange(width, device=lengths.device)
    return (ar.unsqueeze(0) < lengths.reshape(-1, 1)).to(dtype)
