"""LM head fused with the token log-probability (and entropy): the ``[T, V]`` logits are never
materialised for more than one token chunk.

Forward per chunk: ``z = h_c W^T`` -> per-row (max, sum-exp, target logit, sum e^z z) -> combine
over vocabulary shards (one tiny all-gather of 16-byte records instead of the three
all-reduces of the reference, ``mindspeed_rl/utils/compute.py:29-97``) -> ``logp, entropy, lse``.
Backward per chunk: recompute ``z``, overwrite it with ``d loss/d z`` in place, then
``dh_c = dz W`` and ``dW += dz^T h_c``.

CUDA path: GEMMs + ``csrc/logprob.cu`` row kernels; CPU path: PyTorch fp32.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import guard
import torch.distributed as dist

import os

from . import _lib
from . import gemm as _gemm
from ._lib import c_float, c_int, c_ll, check, ptr, stream

DEFAULT_CHUNK = 4096
# MSRL_LMHEAD_TCGEN05=0 selects the chunked cuBLAS + row-kernel formulation (the baseline path)
USE_TCGEN05 = os.environ.get("MSRL_LMHEAD_TCGEN05", "1") != "0"


def _world(group) -> int:
    if group is None or not dist.is_available() or not dist.is_initialized():
        return 1
    return dist.get_world_size(group)


def _combine_stats(stats: torch.Tensor, group) -> Tuple[torch.Tensor, int]:
    """stats ``[T, 4]`` of this shard -> ``[nshard, T, 4]``."""
    ws = _world(group)
    if ws == 1:
        return stats.unsqueeze(0), 1
    out = guard.empty(ws, *stats.shape, device=stats.device, dtype=stats.dtype)
    dist.all_gather_into_tensor(out.view(-1), stats.view(-1).contiguous(), group=group)
    return out, ws


def lmhead_logprob_fwd(h: torch.Tensor, w: torch.Tensor, labels: torch.Tensor, inv_temp: float = 1.0,
                       vocab_offset: int = 0, group=None, want_entropy: bool = True,
                       chunk: int = DEFAULT_CHUNK
                       ) -> Tuple[torch.Tensor, Optional[torch.Tensor], torch.Tensor]:
    """``h [T, H]``, ``w [V_local, H]``, ``labels [T]`` (global ids) -> ``(logp, entropy, lse)`` fp32."""
    t = h.shape[0]
    v = w.shape[0]
    dev = h.device
    logp = guard.empty(t, device=dev, dtype=torch.float32)
    ent = guard.empty(t, device=dev, dtype=torch.float32) if want_entropy else None
    lse = guard.empty(t, device=dev, dtype=torch.float32)
    labels = labels.to(torch.int64).contiguous()
    if _lib.use_kernels(h, w, labels) and h.dtype == torch.bfloat16:
        L = _lib.load()
        if USE_TCGEN05 and _gemm.tcgen05_usable(h, w):
            # fused path: tcgen05 GEMM whose epilogue reduces each 256-column tile to a 16-byte
            # record per row; the [T, V] logits are never written
            stats, tiles = _gemm.lmhead_stats(h, w, labels, inv_temp, vocab_offset)
            if _world(group) > 1:
                m = stats[..., 0].max(dim=0).values
                c = torch.exp(stats[..., 0] - m)
                local = torch.stack([m, (stats[..., 1] * c).sum(0), stats[..., 2].sum(0),
                                     (stats[..., 3] * c).sum(0)], dim=-1).contiguous()
                stats, tiles = _combine_stats(local, group)
            check(L.msrl_logprob_finish(ptr(stats), c_int(tiles), c_ll(t), ptr(logp),
                                        ptr(ent) if ent is not None else None, ptr(lse), stream()),
                  "logprob_finish")
            return logp, ent, lse
        for s in range(0, t, chunk):
            e = min(t, s + chunk)
            z = _gemm.linear_fwd(h[s:e], w)                      # [c, V] bf16
            st = guard.empty(e - s, 4, device=dev, dtype=torch.float32)
            check(L.msrl_logprob_stats(ptr(z), c_ll(z.stride(0)), c_ll(e - s), c_int(v),
                                       c_int(vocab_offset), ptr(labels[s:e]), c_float(inv_temp),
                                       ptr(st), stream()), "logprob_stats")
            allst, ns = _combine_stats(st, group)
            check(L.msrl_logprob_finish(ptr(allst), c_int(ns), c_ll(e - s), ptr(logp[s:e]),
                                        ptr(ent[s:e]) if ent is not None else None, ptr(lse[s:e]),
                                        stream()), "logprob_finish")
        return logp, ent, lse
    for s in range(0, t, chunk):
        e = min(t, s + chunk)
        z = torch.matmul(h[s:e].float(), w.float().t()) * inv_temp
        m = z.max(dim=-1).values
        ez = torch.exp(z - m.unsqueeze(-1))
        y = labels[s:e] - vocab_offset
        mine = (y >= 0) & (y < v)
        zy = torch.where(mine, z.gather(-1, y.clamp(0, v - 1).unsqueeze(-1)).squeeze(-1),
                         torch.zeros_like(m))
        st = torch.stack([m, ez.sum(-1), zy, (ez * z).sum(-1)], dim=-1).contiguous()
        allst, ns = _combine_stats(st, group)
        gm = allst[..., 0].max(dim=0).values
        c = torch.exp(allst[..., 0] - gm)
        ssum = (allst[..., 1] * c).sum(0)
        spz = (allst[..., 3] * c).sum(0)
        l = gm + torch.log(ssum)
        logp[s:e] = allst[..., 2].sum(0) - l
        lse[s:e] = l
        if ent is not None:
            ent[s:e] = l - spz / ssum
    return logp, ent, lse


def lmhead_logprob_bwd(h: torch.Tensor, w: torch.Tensor, labels: torch.Tensor, lse: torch.Tensor,
                       entropy: Optional[torch.Tensor], dlogp: torch.Tensor,
                       dent: Optional[torch.Tensor], dw_accum: Optional[torch.Tensor],
                       inv_temp: float = 1.0, vocab_offset: int = 0,
                       chunk: int = DEFAULT_CHUNK) -> torch.Tensor:
    """Returns this shard's contribution to ``dh`` (sum over vocabulary shards is the caller's
    reduction) and accumulates ``dW`` into ``dw_accum`` (same shape as ``w``; may be ``None``)."""
    t = h.shape[0]
    v = w.shape[0]
    dh = guard.empty_like(h)
    labels = labels.to(torch.int64).contiguous()
    dlogp = dlogp.float().contiguous()
    dent = dent.float().contiguous() if dent is not None else None
    if _lib.use_kernels(h, w, labels) and h.dtype == torch.bfloat16:
        L = _lib.load()
        for s in range(0, t, chunk):
            e = min(t, s + chunk)
            z = _gemm.linear_fwd(h[s:e], w)
            check(L.msrl_logprob_bwd(ptr(z), c_ll(z.stride(0)), c_ll(e - s), c_int(v),
                                     c_int(vocab_offset), ptr(labels[s:e]), c_float(inv_temp),
                                     ptr(lse[s:e]), ptr(entropy[s:e]) if dent is not None else None,
                                     ptr(dlogp[s:e]), ptr(dent[s:e]) if dent is not None else None,
                                     stream()), "logprob_bwd")
            if _gemm._pair_pays(e - s, h.shape[1]) and _gemm.pair_usable(z, w):
                _gemm.gemm_pair(z, w, b_mn=True, out=dh[s:e])
            else:
                torch.matmul(z, w, out=dh[s:e])
            if dw_accum is not None:
                _gemm.linear_wgrad_(dw_accum, z, h[s:e])
        return dh
    for s in range(0, t, chunk):
        e = min(t, s + chunk)
        hf = h[s:e].float()
        z = torch.matmul(hf, w.float().t()) * inv_temp
        p = torch.exp(z - lse[s:e].unsqueeze(-1))
        dz = -dlogp[s:e].unsqueeze(-1) * p
        y = labels[s:e] - vocab_offset
        mine = (y >= 0) & (y < v)
        rows = torch.nonzero(mine).squeeze(-1)
        dz[rows, y[rows]] += dlogp[s:e][rows]
        if dent is not None:
            mean_z = (lse[s:e] - entropy[s:e]).unsqueeze(-1)
            dz = dz + dent[s:e].unsqueeze(-1) * p * (mean_z - z)
        dz = dz * inv_temp
        dh[s:e] = torch.matmul(dz, w.float()).to(h.dtype)
        if dw_accum is not None:
            dw_accum.add_(torch.matmul(dz.t(), hf).to(dw_accum.dtype))
    return dh
