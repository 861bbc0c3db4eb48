"""Rollout-engine ops: paged KV-cache write / gather, paged decode attention, token sampler.

Cache tensors are ``[num_blocks, block_size, n_kv_heads, head_dim]``.  CUDA path:
``csrc/decode.cu``.  The CPU path keeps the same semantics in plain PyTorch so the engine and
its scheduler can be exercised without a GPU.
"""
from __future__ import annotations

import ctypes
import math
import os
from typing import Optional, Sequence, Tuple

import torch

from . import guard

from . import _lib
from ._lib import c_float, c_int, c_ll, c_ull, check, ptr, stream
from .elementwise import _workspace
from .gemm import _status_word
from .layouts import QKVLayout


def _lay(*specs):
    vals = []
    for _, (st, gs, hpg, hs) in specs:
        vals += [st, gs, hpg, hs]
    return (ctypes.c_longlong * len(vals))(*vals)


def kv_cache_write(qkv: torch.Tensor, layout: QKVLayout, slots: torch.Tensor,
                   k_cache: torch.Tensor, v_cache: torch.Tensor) -> None:
    """Store the k / v heads of each row of ``qkv`` at ``slots[t]`` (int64; < 0 skips the row)."""
    t = qkv.shape[0]
    nkv, hd = layout.num_kv_heads, layout.head_dim
    if _lib.use_kernels(qkv, slots, k_cache):
        flat = qkv.view(-1)
        ks, vs = layout.k(), layout.v()
        check(_lib.load().msrl_kv_cache_write(ptr(flat[ks[0]:]), ptr(flat[vs[0]:]), _lay(ks, vs),
                                              ptr(slots), ptr(k_cache), ptr(v_cache), c_ll(t),
                                              c_int(nkv), c_int(hd), stream()), "kv_cache_write")
        return
    _, k, v = layout.split(qkv)
    ok = slots >= 0
    kc = k_cache.view(-1, nkv, hd)
    vc = v_cache.view(-1, nkv, hd)
    kc[slots[ok]] = k[ok].to(kc.dtype)
    vc[slots[ok]] = v[ok].to(vc.dtype)


def kv_cache_gather(k_cache: torch.Tensor, v_cache: torch.Tensor, block_tables: torch.Tensor,
                    token_seq: torch.Tensor, token_pos: torch.Tensor
                    ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Contiguous ``[T, nkv, hd]`` K / V for tokens given as (block-table row, position)."""
    nb, bs, nkv, hd = k_cache.shape
    t = token_seq.numel()
    if _lib.use_kernels(k_cache, block_tables, token_seq):
        k = guard.empty(t, nkv, hd, device=k_cache.device, dtype=k_cache.dtype)
        v = guard.empty_like(k)
        check(_lib.load().msrl_kv_cache_gather(ptr(k_cache), ptr(v_cache), ptr(block_tables),
                                               c_int(block_tables.shape[1]), ptr(token_seq),
                                               ptr(token_pos), ptr(k), ptr(v), c_ll(t), c_int(nkv),
                                               c_int(hd), c_int(bs), stream()), "kv_cache_gather")
        return k, v
    blk = block_tables[token_seq.long(), (token_pos // bs).long()].long()
    slot = blk * bs + (token_pos % bs).long()
    return k_cache.view(-1, nkv, hd)[slot], v_cache.view(-1, nkv, hd)[slot]


def decode_prefix_tile(num_heads: int, num_kv_heads: int, head_dim: int, block_size: int) -> int:
    """Key tile of the tcgen05 shared-prefix kernel for this shape, or 0 when the shape is served by
    the ``mma.sync`` kernel (other head sizes, block sizes that do not divide the tile, no GPU library,
    ``MSRL_PREFIX_TCGEN05=0``).  With a non-zero tile the groups' shared prefix must be rounded down to
    a multiple of it (``build_decode_groups(..., multiple=tile)``)."""
    if os.environ.get("MSRL_PREFIX_TCGEN05", "1") != "1" or not torch.cuda.is_available() or not _lib.available():
        return 0
    return int(_lib.load().msrl_paged_prefix_tcgen05_tile(c_int(num_heads), c_int(num_kv_heads), c_int(head_dim),
                                                          c_int(block_size)))


def decode_group_max(num_heads: int, num_kv_heads: int, prefix_tile: int = 0) -> int:
    """Largest group the shared-prefix decode kernel serves with one CTA: members x query heads per
    KV head must fit the kernel's query rows (128 on the tcgen05 kernel, 64 on the ``mma.sync`` one)."""
    rows = 128 if prefix_tile else 64
    return max(1, min(8, rows // max(num_heads // num_kv_heads, 1)))


def build_decode_groups(group_ids: Sequence, prefix_lens: Sequence[int], group_max: int, multiple: int = 1):
    """Host-side grouping for the shared-prefix decode path.

    ``group_ids[i]`` identifies the prompt of batch row ``i`` and ``prefix_lens[i]`` the number of
    leading tokens it shares with the other rows of that prompt.  Returns
    ``(key_start [B], group_rows [B][8], group_prefix [B], any_shared)`` as python lists padded to
    ``B`` groups (unused groups have first member -1), so the arrays have a fixed shape per batch
    size (CUDA-graph friendly); groups with members come first.  ``multiple`` rounds every shared prefix
    down to a multiple of that many keys (the remainder is then read per sequence).
    """
    b = len(group_ids)
    by_id = {}
    for i, gid in enumerate(group_ids):
        by_id.setdefault(gid, []).append(i)
    key_start = [0] * b
    rows_out, prefix_out = [], []
    shared = False
    for members in by_id.values():
        for s in range(0, len(members), group_max):
            chunk = members[s:s + group_max]
            prefix = min(prefix_lens[i] for i in chunk) if len(chunk) > 1 else 0
            prefix = prefix // multiple * multiple
            shared = shared or prefix > 0
            for i in chunk:
                key_start[i] = prefix
            rows_out.append(chunk + [-1] * (8 - len(chunk)))
            prefix_out.append(prefix)
    while len(rows_out) < b:
        rows_out.append([-1] * 8)
        prefix_out.append(0)
    return key_start, rows_out, prefix_out, shared


def _prefix_splits(n_groups: int, nkv: int, device, per_sm: int) -> int:
    """Splits of the shared prompt per (group, KV head): as many as fill one wave of the prefix kernel
    (``per_sm`` CTAs per SM); ``MSRL_PREFIX_SPLITS`` overrides."""
    env = os.environ.get("MSRL_PREFIX_SPLITS")
    if env:
        return max(1, min(8, int(env)))
    slots = per_sm * torch.cuda.get_device_properties(device).multi_processor_count
    return max(1, min(8, slots // max(1, n_groups * nkv)))


def paged_decode_attention(qkv: torch.Tensor, layout: QKVLayout, k_cache: torch.Tensor,
                           v_cache: torch.Tensor, block_tables: torch.Tensor,
                           context_lens: torch.Tensor, max_context: int,
                           out: Optional[torch.Tensor] = None,
                           groups: Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None,
                           prefix_splits: Optional[int] = None, prefix_tile: int = 0) -> torch.Tensor:
    """One query token per sequence against its paged KV (which already holds that token).

    ``groups = (key_start [B], group_rows [G, 8], group_prefix [G])`` (int32, device) enables the
    shared-prefix path: the members of a group (the n samples of one prompt) have identical
    first ``group_prefix`` tokens, whose K/V is then read once per group instead of once per
    member.  Every row must belong to exactly one group; the result is the same either way.  The group
    tables may list fewer groups than rows (the launch covers ``group_rows.shape[0]`` groups).
    ``prefix_tile`` (``decode_prefix_tile``) states that every ``group_prefix`` is a multiple of that many
    keys and sends the shared pass to the tcgen05 kernel.
    """
    b = qkv.shape[0]
    nh, nkv, hd = layout.num_heads, layout.num_kv_heads, layout.head_dim
    bs = k_cache.shape[1]
    if out is None:
        out = guard.empty(b, nh * hd, device=qkv.device, dtype=qkv.dtype)
    if _lib.use_kernels(qkv, k_cache, block_tables, context_lens):
        L = _lib.load()
        nsplit = L.msrl_paged_decode_nsplit(c_int(b), c_int(nkv), c_int(int(max_context)))
        if groups is not None:
            key_start, group_rows, group_prefix = groups
            if prefix_splits is None:
                # tcgen05 kernel: two CTAs per SM; mma.sync kernel: three
                prefix_splits = _prefix_splits(group_rows.shape[0], nkv, qkv.device, 2 if prefix_tile else 3)
            slots = nsplit + prefix_splits
            part_o = _workspace("decode_part_o", b * nh * slots * hd, qkv.device)
            part_ml = _workspace("decode_part_ml", b * nh * slots * 2, qkv.device)
            qs = layout.q()
            check(L.msrl_paged_decode_grouped(
                ptr(qkv.view(-1)[qs[0]:]), _lay(qs), ptr(k_cache), ptr(v_cache), ptr(block_tables),
                c_int(block_tables.shape[1]), ptr(context_lens), ptr(key_start), ptr(group_rows),
                ptr(group_prefix), c_int(group_rows.shape[0]), ptr(out), c_ll(nh * hd), ptr(part_o), ptr(part_ml),
                c_int(b), c_int(nh), c_int(nkv), c_int(hd), c_int(bs), c_int(nsplit), c_int(prefix_splits),
                c_ll(k_cache.shape[0]), c_int(prefix_tile), ptr(_status_word(qkv.device)),
                stream()), "paged_decode_grouped")
            return out
        part_o = _workspace("decode_part_o", b * nh * nsplit * hd, qkv.device)
        part_ml = _workspace("decode_part_ml", b * nh * nsplit * 2, qkv.device)
        qs = layout.q()
        check(L.msrl_paged_decode(ptr(qkv.view(-1)[qs[0]:]), _lay(qs), ptr(k_cache), ptr(v_cache),
                                  ptr(block_tables), c_int(block_tables.shape[1]), ptr(context_lens),
                                  ptr(out), c_ll(nh * hd), ptr(part_o), ptr(part_ml), c_int(b),
                                  c_int(nh), c_int(nkv), c_int(hd), c_int(bs), c_int(nsplit),
                                  stream()), "paged_decode")
        return out
    q, _, _ = layout.split(qkv)
    rep = nh // nkv
    scale = 1.0 / math.sqrt(hd)
    kc, vc = k_cache.view(-1, nkv, hd), v_cache.view(-1, nkv, hd)
    for i in range(b):
        n = int(context_lens[i])
        pos = torch.arange(n, device=qkv.device)
        slot = block_tables[i, (pos // bs).long()].long() * bs + pos % bs
        k = kc[slot].float().repeat_interleave(rep, dim=1)      # [n, nh, hd]
        v = vc[slot].float().repeat_interleave(rep, dim=1)
        s = torch.einsum("hd,nhd->hn", q[i].float(), k) * scale
        p = torch.softmax(s, dim=-1)
        out[i] = torch.einsum("hn,nhd->hd", p, v).reshape(nh * hd).to(out.dtype)
    return out


# ------------------------------------------------------------------------------------------------
# Sampler
# ------------------------------------------------------------------------------------------------
def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: Optional[torch.Tensor],
           top_p: Optional[torch.Tensor], min_p: Optional[torch.Tensor], row_keys: torch.Tensor,
           seed: int, eos_prob: Optional[torch.Tensor] = None, eos_id: int = -1,
           vocab_offset: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Draw one token per row from ``softmax(logits / T)`` after top-k / top-p / min-p filtering.

    ``temperature[b] <= 0`` means greedy.  ``row_keys`` (uint64 as int64) individualise the random
    stream per request and step; together with ``seed`` the draw is reproducible.  ``eos_prob``
    (>= 0) forces the probability of ``eos_id`` (benchmark length control).
    Returns ``(tokens int64 [B], logprobs fp32 [B])`` under the temperature-scaled distribution.
    """
    b, v = logits.shape
    inv_t = torch.where(temperature > 0, 1.0 / temperature.clamp(min=1e-6),
                        torch.zeros_like(temperature)).float()
    need_filter = any(x is not None for x in (top_k, top_p, min_p))
    if _lib.use_kernels(logits, temperature, row_keys):
        L = _lib.load()
        is_bf16 = 1 if logits.dtype == torch.bfloat16 else 0
        if not is_bf16 and logits.dtype != torch.float32:
            logits = logits.float()
        logits = logits if logits.stride(-1) == 1 else logits.contiguous()
        dev = logits.device
        thresh = None
        if need_filter:
            tk = top_k.to(torch.int32) if top_k is not None else torch.zeros(b, dtype=torch.int32, device=dev)
            tp = top_p.float() if top_p is not None else torch.ones(b, device=dev)
            mp = min_p.float() if min_p is not None else torch.zeros(b, device=dev)
            thresh = guard.empty(b, device=dev, dtype=torch.float32)
            check(L.msrl_sample_filter(ptr(logits), c_int(is_bf16), c_ll(logits.stride(0)), c_int(b),
                                       c_int(v), ptr(inv_t), ptr(tk), ptr(tp), ptr(mp), ptr(thresh),
                                       stream()), "sample_filter")
        nsplit = int(L.msrl_sample_nsplit(c_int(b), c_int(v)))      # vocabulary splits per row (one CTA each)
        rec = guard.empty(b * nsplit * L.msrl_sample_rec_bytes(), device=dev, dtype=torch.uint8)
        ep = eos_prob.float() if eos_prob is not None else None
        check(L.msrl_sample(ptr(logits), c_int(is_bf16), c_ll(logits.stride(0)), c_int(b), c_int(v),
                            c_int(vocab_offset), ptr(inv_t), ptr(thresh), ptr(ep), c_int(eos_id),
                            ptr(row_keys), c_ull(seed & (2 ** 64 - 1)), ptr(rec), c_int(nsplit), stream()),
              "sample")
        tokens = guard.empty(b, device=dev, dtype=torch.int64)
        logprobs = guard.empty(b, device=dev, dtype=torch.float32)
        check(L.msrl_sample_combine(ptr(rec), c_int(nsplit), c_int(b), ptr(ep), c_int(eos_id), ptr(row_keys),
                                    c_ull(seed & (2 ** 64 - 1)), ptr(tokens), ptr(logprobs), stream()),
              "sample_combine")
        return tokens, logprobs
    return _sample_reference(logits, inv_t, top_k, top_p, min_p, row_keys, seed, eos_prob, eos_id)


def _sample_reference(logits, inv_t, top_k, top_p, min_p, row_keys, seed, eos_prob, eos_id):
    b, v = logits.shape
    z = logits.float() * torch.where(inv_t > 0, inv_t, torch.ones_like(inv_t)).unsqueeze(1)
    keep = torch.ones_like(z, dtype=torch.bool)
    if top_k is not None:
        for i in range(b):
            k = int(top_k[i])
            if 0 < k < v:
                kth = torch.topk(z[i], k).values[-1]
                keep[i] &= z[i] >= kth
    if min_p is not None:
        mx = z.max(dim=1, keepdim=True).values
        thr = mx + torch.log(min_p.float().clamp(min=1e-30)).unsqueeze(1)
        keep &= torch.where(min_p.unsqueeze(1) > 0, z >= thr, torch.ones_like(keep))
    if top_p is not None:
        for i in range(b):
            p = float(top_p[i])
            if 0 < p < 1:
                zi = z[i].masked_fill(~keep[i], float("-inf"))
                srt, idx = torch.sort(zi, descending=True)
                pr = torch.softmax(srt, dim=0)
                cum = torch.cumsum(pr, dim=0)
                cut = int((cum < p).sum().item()) + 1
                m = torch.zeros(v, dtype=torch.bool)
                m[idx[:cut]] = True
                keep[i] &= m
    zf = z.masked_fill(~keep, float("-inf"))
    if eos_prob is not None and eos_id >= 0:
        forced = eos_prob >= 0
        zf[forced, eos_id] = float("-inf")
    lse = torch.logsumexp(zf, dim=1)
    tokens = guard.empty(b, dtype=torch.int64)
    logprobs = guard.empty(b, dtype=torch.float32)
    for i in range(b):
        g = torch.Generator().manual_seed((int(seed) * 1000003 + int(row_keys[i])) % (2 ** 63))
        if inv_t[i] <= 0:
            tok = int(zf[i].argmax())
        else:
            u = torch.rand(v, generator=g).clamp(min=1e-12)
            tok = int((zf[i] - torch.log(-torch.log(u))).argmax())
        lp = float(zf[i, tok] - lse[i])
        if eos_prob is not None and eos_id >= 0 and float(eos_prob[i]) >= 0:
            pe = float(eos_prob[i])
            if float(torch.rand(1, generator=g)) < pe:
                tok, lp = eos_id, math.log(max(pe, 1e-30))
            else:
                lp += math.log(max(1 - pe, 1e-30))
        tokens[i], logprobs[i] = tok, lp
    return tokens.to(logits.device), logprobs.to(logits.device)
