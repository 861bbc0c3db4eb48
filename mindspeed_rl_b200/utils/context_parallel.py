"""Batch slicing for context parallelism and re-assembly of per-token outputs.

Layouts (reference: ``mindspeed_rl/utils/context_parallel.py:6-163``):

* ring ("megatron_cp_algo"), un-packed: the sequence is cut into ``2*cp`` chunks and rank ``r``
  keeps chunks ``r`` and ``2*cp-1-r`` (zig-zag, balances causal work);
* ring, packed: the same zig-zag applied to every packed sub-sequence separately, boundaries
  given by ``cu_seqlens_padded`` (every block length is a multiple of ``2*cp``);
* Ulysses ("ulysses_cp_algo"): contiguous chunk ``r`` of ``cp``.

The gather side restores the global token order with a permutation that is computed from
the layout itself (closed form), on the device -- no host argsort.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

RING = "megatron_cp_algo"
ULYSSES = "ulysses_cp_algo"


def get_ring_degree(config) -> int:
    cp = config.context_parallel_size
    if cp == 1:
        return 1
    algo = config.context_parallel_algo
    if algo == RING:
        return cp
    if algo == ULYSSES:
        return 1
    ulysses = getattr(config, "ulysses_degree_in_cp", None)
    if not ulysses:
        raise ValueError("hybrid context parallel needs ulysses_degree_in_cp")
    ring, rem = divmod(cp, ulysses)
    if ring <= 1 or rem != 0:
        raise ValueError(f"ulysses_degree_in_cp ({ulysses}) must divide context_parallel_size "
                         f"({cp}) with a ring degree > 1")
    return ring


def zigzag_index_packed(cu_seqlens_padded: torch.Tensor, cp_size: int, cp_rank: int
                        ) -> torch.Tensor:
    """Global packed positions owned by ``cp_rank`` (ascending within each half-chunk)."""
    cu = cu_seqlens_padded.to(torch.int64)
    starts, ends = cu[:-1], cu[1:]
    chunk = (ends - starts) // (2 * cp_size)
    pieces = []
    for s, e, c in zip(starts.tolist(), ends.tolist(), chunk.tolist()):
        pieces.append(torch.arange(s + cp_rank * c, s + (cp_rank + 1) * c))
        pieces.append(torch.arange(e - (cp_rank + 1) * c, e - cp_rank * c))
    if not pieces:
        return torch.empty(0, dtype=torch.int64, device=cu.device)
    return torch.cat(pieces).to(cu.device)


def zigzag_index_plain(seq_len: int, cp_size: int, cp_rank: int, device=None) -> torch.Tensor:
    c = seq_len // (2 * cp_size)
    return torch.cat([torch.arange(cp_rank * c, (cp_rank + 1) * c),
                      torch.arange((2 * cp_size - 1 - cp_rank) * c,
                                   (2 * cp_size - cp_rank) * c)]).to(device)


def get_batch_on_this_cp_rank(config, batch: Dict[str, Optional[torch.Tensor]],
                              cu_seqlens_padded: Optional[torch.Tensor] = None,
                              cp_rank: int = 0, cp_size: Optional[int] = None
                              ) -> Tuple[Dict[str, Optional[torch.Tensor]], Optional[torch.Tensor]]:
    """Slice every ``[B, S, ...]`` entry of ``batch`` (except ``attention_mask``) for this rank.

    Returns ``(batch, index)``; ``index`` holds the global positions kept by this rank for the
    ring layouts and is ``None`` for Ulysses / no CP.
    """
    cp_size = cp_size or config.context_parallel_size
    if cp_size <= 1:
        return batch, None
    algo = config.context_parallel_algo
    packed_ring = (algo == RING and getattr(config, "reset_attention_mask", False)
                   and getattr(config, "attention_mask_type", "causal") == "causal"
                   and cu_seqlens_padded is not None)
    index = None
    out = dict(batch)
    for key, val in batch.items():
        if key == "attention_mask" or val is None:
            continue
        if algo == ULYSSES:
            out[key] = val.chunk(cp_size, dim=1)[cp_rank].contiguous()
            continue
        if packed_ring:
            if index is None:
                index = zigzag_index_packed(cu_seqlens_padded, cp_size, cp_rank).to(val.device)
        else:
            if index is None:
                index = zigzag_index_plain(val.size(1), cp_size, cp_rank, val.device)
        out[key] = val.index_select(1, index)
    return out, index


def restore_permutation(indices_by_rank: torch.Tensor) -> torch.Tensor:
    """Given the concatenation of every rank's kept positions, return ``perm`` such that
    ``gathered[:, perm]`` is in global order (``perm = inverse(indices)``)."""
    n = indices_by_rank.numel()
    perm = torch.empty(n, dtype=torch.int64, device=indices_by_rank.device)
    perm[indices_by_rank] = torch.arange(n, device=indices_by_rank.device)
    return perm


def _all_gather_cat(t: torch.Tensor, group, dim: int) -> torch.Tensor:
    ws = dist.get_world_size(group)
    parts = [torch.empty_like(t) for _ in range(ws)]
    dist.all_gather(parts, t.detach().contiguous(), group=group)
    parts[dist.get_rank(group)] = t  # keep autograd on the local slice
    return torch.cat(parts, dim=dim)


def gather_cp_outputs(cp_tensor: torch.Tensor, cp_size: int, group=None,
                      cu_seqlens_padded: Optional[torch.Tensor] = None,
                      ring: bool = False) -> torch.Tensor:
    """All-gather ``[B, S/cp]`` per-token outputs over the CP group and restore global order."""
    if cp_size <= 1:
        return cp_tensor
    full = _all_gather_cat(cp_tensor, group, dim=1)
    if not ring:
        return full
    dev = cp_tensor.device
    if cu_seqlens_padded is not None:
        idx = torch.cat([zigzag_index_packed(cu_seqlens_padded, cp_size, r).to(dev)
                         for r in range(cp_size)])
    else:
        idx = torch.cat([zigzag_index_plain(full.size(1), cp_size, r, dev)
                         for r in range(cp_size)])
    return full.index_select(1, restore_permutation(idx))


# names used by callers familiar with the reference helpers
def get_tensor_allgather_cp_with_pack(cp_tensor, cp_size, index, group=None, cu_seqlens_padded=None):
    return gather_cp_outputs(cp_tensor, cp_size, group, cu_seqlens_padded, ring=index is not None)


def get_tensor_allgather_cp_without_pack(cp_tensor, cp_size, index, group=None):
    return gather_cp_outputs(cp_tensor, cp_size, group, None, ring=index is not None)
