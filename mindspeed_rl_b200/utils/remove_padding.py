"""Remove-padding ("THD") packing of a padded batch into one token stream and back.

Contract (reference: ``mindspeed_rl/utils/remove_padding.py:10-136``):

* every sequence is padded up to a multiple of ``align`` (``tp*cp``, or ``2*tp*cp`` for ring
  context parallel) and the padded sequences are concatenated into ``[1, T]``;
* position ids restart at 0 in every padded block;
* ``cu_seqlens_padded`` (int32, ``B+1``) delimits the blocks and is what the varlen attention
  kernel consumes; ``seqlens_in_batch`` are the true lengths;
* un-packing restores ``[B, seq_len, ...]`` and can drop the prompt part so that row ``b``
  starts at position ``prompt_len[b]-1`` (the first position that predicts a response token).

Both directions are single gather/scatter operations on the device (kernel ``pack_tokens`` /
``unpack_tokens`` in ``ops.packing`` when CUDA is available).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch


def packed_layout(seqlens: torch.Tensor, align: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Return (padded lengths, cu_seqlens_padded int32[B+1])."""
    seqlens = seqlens.to(torch.int32)
    padded = (seqlens + (align - 1)) // align * align
    cu = torch.zeros(seqlens.numel() + 1, dtype=torch.int32, device=seqlens.device)
    cu[1:] = torch.cumsum(padded, dim=0)
    return padded, cu


def _block_index(cu: torch.Tensor, total: int):
    """For every packed position: owning sequence and offset within its block."""
    pos = torch.arange(total, device=cu.device, dtype=torch.int64)
    seq = torch.searchsorted(cu[1:].to(torch.int64), pos, right=True)
    off = pos - cu.to(torch.int64)[seq]
    return seq, off


def preprocess_packed_seqs(input_ids: torch.Tensor, labels: torch.Tensor,
                           attention_mask_1d: torch.Tensor, tp_size: int):
    """Padded ``[B, S]`` -> packed ``[1, T]`` ids / position ids / labels.

    Returns ``(ids, position_ids, labels, seqlens_in_batch, cu_seqlens_padded)``.
    """
    if attention_mask_1d.shape != input_ids.shape:
        raise ValueError("attention_mask_1d must have the shape of input_ids")
    seqlens = attention_mask_1d.sum(dim=1, dtype=torch.int32)
    _, cu = packed_layout(seqlens, tp_size)
    total = int(cu[-1].item())
    seq, off = _block_index(cu, total)
    valid = off < seqlens.to(torch.int64)[seq]
    src_col = off.clamp(max=input_ids.size(1) - 1)
    ids = torch.where(valid, input_ids[seq, src_col], torch.zeros_like(input_ids[seq, src_col]))
    lab = torch.where(valid, labels[seq, src_col], torch.zeros_like(labels[seq, src_col]))
    return (ids.unsqueeze(0), off.to(torch.int32).unsqueeze(0), lab.unsqueeze(0), seqlens, cu)


def postprocess_packed_seqs(output: torch.Tensor, seqlens_in_batch: torch.Tensor,
                            cu_seqlens_padded: torch.Tensor, seq_len: int,
                            prompt_length: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Packed ``[1, T, ...]`` -> ``[B, seq_len, ...]`` (zeros in padding positions)."""
    if output.shape[0] != 1:
        raise ValueError("packed tensor must have a leading dimension of 1")
    flat = output[0]
    b = seqlens_in_batch.numel()
    lens = seqlens_in_batch.to(torch.int64)
    start = cu_seqlens_padded[:-1].to(torch.int64)
    if prompt_length is not None:
        trunc = prompt_length.reshape(-1).to(torch.int64) - 1
        cut = trunc < lens
        start = torch.where(cut, start + trunc, start)
        lens = torch.where(cut, lens - trunc - 1, lens)
    j = torch.arange(seq_len, device=flat.device).unsqueeze(0)
    valid = j < lens.unsqueeze(1)
    idx = (start.unsqueeze(1) + j).clamp(max=max(flat.size(0) - 1, 0))
    g = flat[idx.reshape(-1)].reshape(b, seq_len, *flat.shape[1:])
    mask = valid.reshape(b, seq_len, *([1] * (flat.dim() - 1)))
    return torch.where(mask, g, torch.zeros_like(g))
