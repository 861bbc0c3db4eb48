"""Remove-padding packing and un-packing as device kernels (``csrc/packing.cu``).

``pack_tokens`` turns padded ``[B, S]`` ids plus the rows' prompt / response lengths into the packed
token stream the model consumes (ids, next-token labels, restart-per-sequence positions);
``unpack_response`` brings a per-token output (log-prob, entropy, value) back to ``[B, W]`` response
rows.  On CPU tensors both run the equivalent index arithmetic in PyTorch, which is also the
oracle of the kernels (reference behaviour: ``mindspeed_rl/utils/remove_padding.py:55-79,118-134``).
"""
from __future__ import annotations

from typing import Tuple

import torch

from . import guard

from . import _lib
from ._lib import c_int, c_ll, check, ptr, stream


def pack_tokens(ids2d: torch.Tensor, p_len: torch.Tensor, r_len: torch.Tensor, cu: torch.Tensor,
                total: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``ids2d [B, S]`` (int32 / int64), ``p_len`` / ``r_len`` ``[B]`` int32, ``cu [B+1]`` int32 block
    offsets (every block at least as long as its sequence) -> ``(ids [T] int64, labels [T] int64,
    positions [T] int32)``."""
    b, s = ids2d.shape
    dev = ids2d.device
    if _lib.use_kernels(ids2d, p_len, r_len, cu):
        ids2d = ids2d if ids2d.stride(1) == 1 else ids2d.contiguous()
        if ids2d.dtype not in (torch.int32, torch.int64):
            ids2d = ids2d.long()
        out_ids = guard.empty(total, dtype=torch.int64, device=dev)
        out_lab = guard.empty(total, dtype=torch.int64, device=dev)
        out_pos = guard.empty(total, dtype=torch.int32, device=dev)
        check(_lib.load().msrl_pack_tokens(
            ptr(ids2d), c_int(1 if ids2d.dtype == torch.int64 else 0), c_ll(ids2d.stride(0)), ptr(p_len), ptr(r_len),
            ptr(cu), c_int(b), c_int(s), c_ll(total), ptr(out_ids), ptr(out_lab), ptr(out_pos), stream()), "pack_tokens")
        return out_ids, out_lab, out_pos
    cu64 = cu.to(torch.int64)
    lens = (p_len.to(torch.int64) + r_len.to(torch.int64)).clamp(max=s)
    pos = torch.arange(total, device=dev, dtype=torch.int64)
    seq = torch.searchsorted(cu64[1:], pos, right=True).clamp(max=max(b - 1, 0))
    off = pos - cu64[seq]
    src = ids2d.to(torch.int64)
    col = off.clamp(max=s - 1)
    ids = torch.where(off < lens[seq], src[seq, col], torch.zeros_like(off))
    nxt = (off + 1).clamp(max=s - 1)
    labels = torch.where(off + 1 < lens[seq], src[seq, nxt], torch.zeros_like(off))
    return ids, labels, off.to(torch.int32)


def unpack_response(src: torch.Tensor, cu: torch.Tensor, p_len: torch.Tensor, r_len: torch.Tensor,
                    width: int) -> torch.Tensor:
    """``src [T]`` (fp32 / bf16) -> ``[B, width]`` fp32: row ``b`` holds ``src[cu[b] + p_len[b] - 1 + j]``
    for ``j < r_len[b]`` and zeros after."""
    b = p_len.numel()
    if _lib.use_kernels(src, cu, p_len, r_len) and src.dtype in (torch.float32, torch.bfloat16):
        src = src.contiguous()
        out = guard.empty(b, width, dtype=torch.float32, device=src.device)
        check(_lib.load().msrl_unpack_response(
            ptr(src), c_int(1 if src.dtype == torch.bfloat16 else 0), ptr(cu), ptr(p_len), ptr(r_len), c_int(b),
            c_int(width), c_ll(src.numel()), ptr(out), stream()), "unpack_response")
        return out
    j = torch.arange(width, device=src.device).unsqueeze(0)
    idx = (cu[:-1].to(torch.int64) + p_len.to(torch.int64) - 1).unsqueeze(1) + j
    valid = (j < r_len.to(torch.int64).unsqueeze(1)) & (idx >= 0) & (idx < src.numel())
    g = src.float()[idx.clamp(0, max(src.numel() - 1, 0))]
    return torch.where(valid, g, torch.zeros_like(g))
