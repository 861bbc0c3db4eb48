"""Context parallelism: shard every packed sequence over the CP group and run attention on it.

Token split (what each CP rank keeps of a packed stream whose sequences are padded to a multiple
of ``2 * cp``): the *zig-zag* layout of the ring algorithm (chunks ``r`` and ``2cp-1-r`` of every
sequence, which balances causal work; reference ``mindspeed_rl/utils/context_parallel.py:6-163``)
or contiguous chunks for the Ulysses algorithm.  Everything outside attention is token-wise and
runs on the local tokens unchanged.

Attention runs head-parallel: an all-to-all over the CP group turns ``[local tokens, all heads]``
into ``[all tokens, heads / cp]`` (tokens restored to sequence order, so the ordinary packed
causal flash-attention kernel applies with the original ``cu_seqlens``), and a second all-to-all
brings the result back.  This is the Ulysses exchange; it is also used for the zig-zag layout
whenever the (TP-local) KV heads divide by ``cp``, because on one NVSwitch domain an all-to-all of
activations costs the same bytes as the ring's KV rotation without serialising ``cp`` steps.

The ring algorithm proper (``megatron_cp_algo`` when the head counts do not divide by ``cp``, or
``MSRL_CP_RING=1``) keeps all heads local and rotates K/V around the CP group instead: step 0 is
causal attention on the local zig-zag pair of chunks; at step s the K/V of rank ``j = r - s``
arrive (the transfer of step s+1 is posted before the math of step s) and, because of the zig-zag
order, the block is never masked: all local queries against the first chunk of ``j`` when
``j < r``, the queries of the second local chunk against both chunks of ``j`` otherwise.  Block
results are merged with their log-sum-exp.  The backward runs the same rotation, recomputes each
block's probabilities from the merged log-sum-exp, adds dQ locally and returns every block's
dK/dV to the rank that owns those keys (reference: ring attention of
``docs/zh/features/context_parallel.md:52-86``).

``hybrid_cp_algo`` composes the two: ``cp = ring x ulysses``.  Neighbouring ranks form Ulysses
sub-groups of ``ulysses_degree`` members that hold contiguous pieces of one ring position's
zig-zag pair of chunks; an all-to-all inside the sub-group turns them into ``heads / ulysses``
heads of the whole pair, and the ring runs between the sub-groups (members with the same index).

Per-token outputs (log-probs, values) are all-gathered and put back in global order; in the
backward every rank keeps the gradient of its own tokens, scaled by ``cp`` because the
data-parallel averaging that follows divides by ``dp * cp``.
"""
from __future__ import annotations

import os
from typing import Any, List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import ops
from ..ops import QKVLayout

RING, ULYSSES, HYBRID = "megatron_cp_algo", "ulysses_cp_algo", "hybrid_cp_algo"


def split_index(cu_padded: torch.Tensor, cp_size: int, cp_rank: int, zigzag: bool) -> torch.Tensor:
    """Global packed positions kept by ``cp_rank`` (int64, host), ascending within each piece."""
    cu = cu_padded.to(torch.int64).tolist()
    pieces = []
    for s, e in zip(cu[:-1], cu[1:]):
        n = e - s
        if zigzag:
            c = n // (2 * cp_size)
            if c * 2 * cp_size != n:
                raise ValueError(f"sequence length {n} is not a multiple of 2*cp = {2 * cp_size}")
            pieces.append(torch.arange(s + cp_rank * c, s + (cp_rank + 1) * c))
            pieces.append(torch.arange(e - (cp_rank + 1) * c, e - cp_rank * c))
        else:
            c = n // cp_size
            if c * cp_size != n:
                raise ValueError(f"sequence length {n} is not a multiple of cp = {cp_size}")
            pieces.append(torch.arange(s + cp_rank * c, s + (cp_rank + 1) * c))
    return torch.cat(pieces) if pieces else torch.empty(0, dtype=torch.int64)


class _GatherTokens(torch.autograd.Function):
    """[T_local, ...] -> [T, ...] in global order; backward keeps the local rows (x cp)."""

    @staticmethod
    def forward(ctx, x, cp: "ContextParallel"):
        ctx.cp = cp
        parts = [torch.empty_like(x) for _ in range(cp.size)]
        dist.all_gather(parts, x.contiguous(), group=cp.group)
        return torch.cat(parts, 0)[cp.restore]

    @staticmethod
    def backward(ctx, d):
        cp = ctx.cp
        return d[cp.local_index_dev] * float(cp.size), None


_sub_groups = {}


def hybrid_sub_groups(group, size: int, rank: int, ulysses: int):
    """``(ring group, ulysses group)`` of this rank for ``cp = ring x ulysses`` (created once per CP
    group; only the members of a sub-group take part in its creation)."""
    members = dist.get_process_group_ranks(group)
    key = (tuple(members), ulysses)
    if key not in _sub_groups:
        ring_n = size // ulysses
        mine_ring = mine_uly = None
        for j in range(ulysses):                   # ring groups: same index inside the ulysses sub-group
            ranks = [members[i * ulysses + j] for i in range(ring_n)]
            if members[rank] in ranks:
                mine_ring = dist.new_group(ranks, use_local_synchronization=True)
        for i in range(ring_n):                    # ulysses groups: neighbouring ranks
            ranks = members[i * ulysses:(i + 1) * ulysses]
            if members[rank] in ranks:
                mine_uly = dist.new_group(ranks, use_local_synchronization=True)
        _sub_groups[key] = (mine_ring, mine_uly)
    return _sub_groups[key]


class ContextParallel:
    def __init__(self, group, size: int, rank: int, algo: str, cu_padded: torch.Tensor, device,
                 ulysses_degree: int = 1):
        self.group, self.size, self.rank, self.algo = group, size, rank, algo or RING
        self.device = torch.device(device)
        self.cu_full = cu_padded.to(torch.int32)
        zigzag = self.algo != ULYSSES
        self.outer = self.inner = None
        if self.algo == HYBRID:
            u = max(int(ulysses_degree or 1), 1)
            if size % u:
                raise ValueError(f"ulysses_degree_in_cp {u} must divide the context-parallel size {size}")
            ring_n = size // u
            ring_group, uly_group = hybrid_sub_groups(group, size, rank, u)
            self.outer = ContextParallel(ring_group, ring_n, rank // u, RING, cu_padded, device)
            cu_ring = self.outer.cu_local.cpu().to(torch.int64)
            self.inner = ContextParallel(uly_group, u, rank % u, ULYSSES, cu_ring, device)
            per_rank = []
            for k in range(size):
                ring_tokens = split_index(cu_padded.cpu(), ring_n, k // u, True)
                per_rank.append(ring_tokens[split_index(cu_ring, u, k % u, False)])
        else:
            per_rank = [split_index(cu_padded.cpu(), size, r, zigzag) for r in range(size)]
        self.local_index = per_rank[rank]
        order = torch.cat(per_rank)                     # rank-major order -> global position
        restore = torch.empty_like(order)
        restore[order] = torch.arange(order.numel())
        self.order_dev = order.to(self.device)          # gathered[i] is global token order[i]
        self.restore = restore.to(self.device)          # gathered[restore] is in global order
        self.local_index_dev = self.local_index.to(self.device)
        lens = (cu_padded[1:] - cu_padded[:-1]).to(torch.int64) // size
        cu_local = torch.zeros(lens.numel() + 1, dtype=torch.int32)
        cu_local[1:] = torch.cumsum(lens, 0)
        self.cu_local = cu_local.to(self.device)
        self.max_local = int(lens.max()) if lens.numel() else 0
        self.max_full = int((cu_padded[1:] - cu_padded[:-1]).max()) if lens.numel() else 0
        self.cu_full_dev = self.cu_full.to(self.device)
        self._ring_ready = False

    # ---- ring attention --------------------------------------------------------------------------------
    def use_ring(self, lay: QKVLayout) -> bool:
        if self.algo != RING:
            return False
        return bool(lay.num_kv_heads % self.size or lay.num_heads % self.size) or \
            os.environ.get("MSRL_CP_RING", "0") == "1"

    def _ring_setup(self) -> None:
        if self._ring_ready:
            return
        cu = self.cu_local.cpu().to(torch.int64)
        lens = cu[1:] - cu[:-1]
        half = lens // 2
        first = [torch.arange(int(s), int(s + h)) for s, h in zip(cu[:-1], half)]
        second = [torch.arange(int(s + h), int(e)) for s, h, e in zip(cu[:-1], half, cu[1:])]
        empty = torch.empty(0, dtype=torch.int64)
        self.first_idx = (torch.cat(first) if first else empty).to(self.device)
        self.second_idx = (torch.cat(second) if second else empty).to(self.device)
        cu_half = torch.zeros(lens.numel() + 1, dtype=torch.int32)
        cu_half[1:] = torch.cumsum(half, 0)
        self.cu_half = cu_half.to(self.device)
        self.max_half = int(half.max()) if half.numel() else 0
        self._ring_ready = True

    def _post(self, sends, recvs):
        """``sends`` / ``recvs``: lists of ``(tensor, cp rank)``; returns the requests."""
        ranks = dist.get_process_group_ranks(self.group)
        ops_ = [dist.P2POp(dist.isend, t, ranks[r % self.size], self.group) for t, r in sends] + \
               [dist.P2POp(dist.irecv, t, ranks[r % self.size], self.group) for t, r in recvs]
        return dist.batch_isend_irecv(ops_) if ops_ else []

    @staticmethod
    def _wait(reqs) -> None:
        for q_ in reqs:
            q_.wait()

    def _ring_fwd(self, q, k, v):
        self._ring_setup()
        n, r = self.size, self.rank
        tl, nh, hd = q.shape
        cur = torch.stack([k, v]).contiguous()
        nxt = torch.empty_like(cur) if n > 1 else None
        reqs = self._post([(cur, r + 1)], [(nxt, r - 1)]) if n > 1 else []     # K/V for step 1 travel during step 0
        o, lse = ops.attn_kv_fwd(q, k, v, self.cu_local, self.cu_local, self.max_local, True)
        acc_o, acc_l = o.float().view(tl, nh, hd).contiguous(), lse.clone()    # [Tl, nh, hd], [nh, Tl]
        for s in range(1, n):
            self._wait(reqs)
            cur = nxt                                      # K/V of rank j
            j = (r - s) % n
            if s + 1 < n:
                nxt = torch.empty_like(cur)
                reqs = self._post([(cur, r + 1)], [(nxt, r - 1)])
            if j < r:
                kj, vj = cur[0][self.first_idx], cur[1][self.first_idx]
                o, l = ops.attn_kv_fwd(q, kj, vj, self.cu_local, self.cu_half, self.max_local, False)
                ops.attn_merge_(acc_o, acc_l, o, l)
            else:
                idx = self.second_idx
                o, l = ops.attn_kv_fwd(q[idx], cur[0], cur[1], self.cu_half, self.cu_local, self.max_half, False)
                ops.attn_merge_(acc_o, acc_l, o, l, idx)
        return acc_o.reshape(tl, nh * hd).to(q.dtype), acc_l

    def _ring_bwd(self, dout, q, k, v, out, lse):
        n, r = self.size, self.rank
        tl, nh, hd = q.shape
        dq = torch.zeros(tl, nh, hd, dtype=torch.float32, device=q.device)
        dkv = torch.zeros(2, *k.shape, dtype=torch.float32, device=q.device)
        cur = torch.stack([k, v]).contiguous()
        nxt = torch.empty_like(cur) if n > 1 else None
        reqs = self._post([(cur, r + 1)], [(nxt, r - 1)]) if n > 1 else []
        g = ops.attn_kv_bwd(dout, q, k, v, out, lse, self.cu_local, self.cu_local, self.max_local, self.max_local, True)
        dq += g[0].float()
        dkv[0] += g[1].float()
        dkv[1] += g[2].float()
        home = []                                          # (requests, receive buffer) of dK/dV blocks on their way
        for s in range(1, n):
            self._wait(reqs)
            cur = nxt
            j = (r - s) % n
            if s + 1 < n:
                nxt = torch.empty_like(cur)
                reqs = self._post([(cur, r + 1)], [(nxt, r - 1)])
            part = torch.zeros(2, *k.shape, dtype=k.dtype, device=q.device)
            if j < r:
                idx = self.first_idx
                g = ops.attn_kv_bwd(dout, q, cur[0][idx], cur[1][idx], out, lse, self.cu_local, self.cu_half,
                                    self.max_local, self.max_half, False)
                dq += g[0].float()
                part[0][idx] = g[1]
                part[1][idx] = g[2]
            else:
                idx = self.second_idx
                g = ops.attn_kv_bwd(dout[idx], q[idx], cur[0], cur[1], out[idx], lse[:, idx].contiguous(), self.cu_half,
                                    self.cu_local, self.max_half, self.max_local, False)
                dq[idx] += g[0].float()
                part[0] = g[1]
                part[1] = g[2]
            # this block's dK/dV goes to the rank that owns the keys; mine comes from rank r + s
            back = torch.empty_like(part)
            home.append((self._post([(part, r - s)], [(back, r + s)]), back, part))
        for rq, back, _ in home:
            self._wait(rq)
            dkv += back.float()
        return dq.to(q.dtype), dkv[0].to(k.dtype), dkv[1].to(v.dtype)

    # ---- token plumbing -----------------------------------------------------------------------------
    def take_local(self, t: torch.Tensor) -> torch.Tensor:
        return t[self.local_index_dev.to(t.device)]

    def gather_tokens(self, x_local: torch.Tensor) -> torch.Tensor:
        if torch.is_grad_enabled() and x_local.requires_grad:
            return _GatherTokens.apply(x_local, self)
        return _GatherTokens.forward(_Dummy(), x_local, self)

    # ---- attention ------------------------------------------------------------------------------------
    def _a2a(self, x: torch.Tensor, to_heads: bool) -> torch.Tensor:
        """``to_heads``: [T_local, H, d] -> [T_full (global order), H/cp, d]; else the inverse."""
        c = self.size
        if to_heads:
            tl, h, d = x.shape
            send = x.reshape(tl, c, h // c, d).permute(1, 0, 2, 3).contiguous()     # [c, T_l, H/c, d]
            recv = torch.empty_like(send)
            dist.all_to_all_single(recv, send, group=self.group)
            return recv.reshape(c * tl, h // c, d)[self.restore]
        t, hc, d = x.shape
        tl = t // c
        send = x[self.order_dev].reshape(c, tl, hc, d).contiguous()                # rank-major token blocks
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.group)
        return recv.permute(1, 0, 2, 3).reshape(tl, c * hc, d)

    def _head_layout(self, lay: QKVLayout) -> QKVLayout:
        if lay.num_kv_heads % self.size or lay.num_heads % self.size:
            raise NotImplementedError(
                f"context parallel size {self.size} must divide the local head counts "
                f"({lay.num_heads} query / {lay.num_kv_heads} key-value heads)")
        return QKVLayout(lay.num_heads // self.size, lay.num_kv_heads // self.size, lay.head_dim, interleaved=False)

    def _hybrid_fwd(self, qkv: torch.Tensor, lay: QKVLayout):
        inner, outer = self.inner, self.outer
        inner._head_layout(lay)                           # the ulysses degree must divide the head counts
        q, k, v = (inner._a2a(t.contiguous(), True).contiguous() for t in lay.split(qkv))
        out, lse = outer._ring_fwd(q, k, v)
        tr = q.shape[0]
        back = inner._a2a(out.view(tr, q.shape[1], lay.head_dim), False)
        return back.reshape(qkv.shape[0], lay.num_heads * lay.head_dim), ("hybrid", q, k, v, lse, out)

    def _hybrid_bwd(self, dattn: torch.Tensor, saved, lay: QKVLayout) -> torch.Tensor:
        _, q, k, v, lse, out = saved
        inner, outer = self.inner, self.outer
        tl = dattn.shape[0]
        d_out = inner._a2a(dattn.reshape(tl, lay.num_heads, lay.head_dim).contiguous(), True)
        dq, dk, dv = outer._ring_bwd(d_out.reshape(d_out.shape[0], -1).contiguous(), q, k, v, out, lse)
        dq, dk, dv = (inner._a2a(t.contiguous(), False) for t in (dq, dk, dv))
        return lay.merge(dq, dk, dv)

    def attention_fwd(self, qkv: torch.Tensor, lay: QKVLayout, meta) -> Tuple[torch.Tensor, Any]:
        if self.algo == HYBRID:
            return self._hybrid_fwd(qkv, lay)
        if self.use_ring(lay):
            q, k, v = (t.contiguous() for t in lay.split(qkv))
            out, lse = self._ring_fwd(q, k, v)
            return out, ("ring", q, k, v, lse)
        hl = self._head_layout(lay)
        q, k, v = lay.split(qkv)
        # GQA: query heads of a KV group must land on the rank that gets that KV head
        qf, kf, vf = self._a2a(q.contiguous(), True), self._a2a(k.contiguous(), True), self._a2a(v.contiguous(), True)
        t = qf.shape[0]
        packed = torch.cat([qf, kf, vf], dim=1).reshape(t, hl.width).contiguous()
        out, lse = ops.attn_varlen_fwd(packed, hl, self.cu_full_dev, self.max_full, causal=True)
        back = self._a2a(out.view(t, hl.num_heads, hl.head_dim), False)
        return back.reshape(qkv.shape[0], lay.num_heads * lay.head_dim), (packed, out, lse, hl)

    def attention_bwd(self, dattn: torch.Tensor, qkv: torch.Tensor, attn: torch.Tensor, saved: Any, lay: QKVLayout,
                      meta) -> torch.Tensor:
        if saved[0] == "hybrid":
            return self._hybrid_bwd(dattn, saved, lay)
        if saved[0] == "ring":
            _, q, k, v, lse = saved
            dq, dk, dv = self._ring_bwd(dattn.contiguous(), q, k, v, attn, lse)
            return lay.merge(dq, dk, dv)
        packed, out, lse, hl = saved
        tl = qkv.shape[0]
        d_out = self._a2a(dattn.reshape(tl, lay.num_heads, lay.head_dim).contiguous(), True)
        t = d_out.shape[0]
        d_packed = ops.attn_varlen_bwd(d_out.reshape(t, -1).contiguous(), packed, out, lse, hl, self.cu_full_dev,
                                       self.max_full, causal=True)
        dq, dk, dv = hl.split(d_packed)
        dq, dk, dv = self._a2a(dq.contiguous(), False), self._a2a(dk.contiguous(), False), self._a2a(dv.contiguous(), False)
        return lay.merge(dq, dk, dv)


class _Dummy:
    """Stand-in autograd context for the no-grad path of ``_GatherTokens``."""
