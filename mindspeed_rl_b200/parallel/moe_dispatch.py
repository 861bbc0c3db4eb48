"""Expert-parallel token dispatch / combine over peer-mapped memory (``csrc/moe_p2p.cu``).

``P2PDispatcher`` owns three symmetric-arena buffers shared by all MoE layers: the count table,
the receive slab (token rows grouped by local expert, 128-row padded segments) and the output slab
the source ranks pull from.  One forward of a layer is

    route = d.dispatch(x, expert_ids)            # publish counts | barrier | layout | peer stores | barrier
    y = experts(d.slab, route.plan)              # grouped GEMMs on the slab, result into d.out_slab
    out, rows = d.combine(route, weights)        # barrier | peer loads + weighted sum

and the backward runs the same route with gradients (``dispatch(dout, ..., scale=weights)`` and
``combine(route, None)``).  Without an arena (CPU, several nodes) the MoE layer keeps using the
all-to-all collectives.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch

from ..ops import _lib, guard
from ..ops import moe as K
from ..ops._lib import c_int, c_ll, check, ptr, stream
from .symm import SymmetricArena


@dataclass
class Route:
    plan: K.MoePlan            # destination-side plan of this rank's slab (for the grouped GEMMs)
    slot_rank: torch.Tensor    # [T*k] int32 destination rank (position in the EP team) of every slot
    slot_row: torch.Tensor     # [T*k] int32 row inside that rank's slab
    tokens: int
    k: int


class P2PDispatcher:
    def __init__(self, arena: SymmetricArena, ranks: Sequence[int], experts_local: int, hidden: int, cap_rows: int,
                 dtype: torch.dtype = torch.bfloat16, fallback: bool = True):
        """``ranks``: positions of the expert-parallel group's members inside the arena's team (this
        rank included), in expert order; ``cap_rows``: rows of the slabs (multiple of 128), the same
        on every rank.  ``fallback``: a routing so skewed that some member's slab would overflow makes
        ``dispatch`` return ``None`` on every member (the caller then takes the all-to-all path for that
        call) at the price of one small device-to-host read per call; without it the overflow is
        recorded in the arena's status word and raised at the next stage boundary."""
        if dtype != torch.bfloat16 or hidden % 8:
            raise ValueError("the peer-memory dispatcher moves bf16 rows whose length is a multiple of 8")
        self.arena, self.ranks = arena, list(ranks)
        self.ep = len(self.ranks)
        self.me = self.ranks.index(arena.rank)
        self.e_local, self.hidden = experts_local, hidden
        self.n_total = self.ep * experts_local
        self.cap_rows = (cap_rows + K.PAD - 1) // K.PAD * K.PAD
        if self.ep > int(arena.lib.msrl_moe_p2p_max_ranks()) or self.n_total > 1024:
            raise ValueError("expert-parallel group too large for the peer-memory dispatcher")
        self.table = arena.alloc((self.ep, self.n_total), torch.int32)
        self.slab = arena.alloc((self.cap_rows, hidden), dtype)
        self.out_slab = arena.alloc((self.cap_rows, hidden), dtype)
        dev = self.slab.device
        self.my_base = guard.empty(self.n_total, dtype=torch.int32, device=dev)
        self.fallback = fallback
        self.over = torch.zeros(1, dtype=torch.int32, device=dev)
        self.overflows = 0          # calls that left the peer-memory path
        self._table_ptrs = arena.peer_ptrs(arena.offset_of(self.table), self.ranks)
        self._slab_ptrs = arena.peer_ptrs(arena.offset_of(self.slab), self.ranks)
        self._out_ptrs = arena.peer_ptrs(arena.offset_of(self.out_slab), self.ranks)
        self.calls = 0

    @staticmethod
    def bytes_needed(ep: int, experts_local: int, hidden: int, cap_rows: int) -> int:
        cap = (cap_rows + K.PAD - 1) // K.PAD * K.PAD
        return ep * ep * experts_local * 4 + 2 * cap * hidden * 2 + 3 * 256

    def dispatch(self, x: torch.Tensor, expert_ids: torch.Tensor, scale: Optional[torch.Tensor] = None,
                 route: Optional[Route] = None) -> Optional[Route]:
        """Send ``x[t]`` (times ``scale[t, j]``) to the rank of expert ``expert_ids[t, j]`` (global
        ids).  Returns ``None`` (on every member alike, nothing sent) when a slab would overflow and
        ``fallback`` is on."""
        lib, st = self.arena.lib, stream()
        t, k = expert_ids.shape
        dev = x.device
        x = x.contiguous()
        flat = expert_ids.reshape(-1).contiguous()
        plan_src = K.moe_plan(expert_ids, self.n_total)          # per-expert counts and stable ranks of my slots
        check(lib.msrl_moe_p2p_publish(self._table_ptrs, ptr(plan_src.counts), c_int(self.n_total), c_int(self.me),
                                       c_int(self.ep), st), "moe_p2p_publish")
        self.arena.barrier(self.ranks)
        # the verdict is read on the host, which a stream capture (decode steps replayed from a CUDA graph)
        # does not allow: there the overflow goes to the status word and is raised at the stage boundary
        ask = self.fallback and not torch.cuda.is_current_stream_capturing()
        counts_l = guard.empty(self.e_local, dtype=torch.int32, device=dev)
        offsets_l = guard.empty(self.e_local + 1, dtype=torch.int32, device=dev)
        tiles = guard.empty(self.cap_rows // K.PAD, dtype=torch.int32, device=dev)
        check(lib.msrl_moe_p2p_layout(ptr(self.table), c_int(self.ep), c_int(self.e_local), c_int(self.me),
                                      c_int(self.cap_rows), ptr(self.my_base), ptr(counts_l), ptr(offsets_l),
                                      ptr(tiles), None if ask else ptr(self.arena.status),
                                      ptr(self.over) if ask else None, st), "moe_p2p_layout")
        if ask and int(self.over.item()):
            self.over.zero_()
            self.overflows += 1
            return None
        slot_rank = guard.empty(t * k, dtype=torch.int32, device=dev)
        slot_row = guard.empty(t * k, dtype=torch.int32, device=dev)
        wf = None if scale is None else scale.reshape(-1).float().contiguous()
        check(lib.msrl_moe_p2p_dispatch(ptr(x), c_ll(x.shape[1]), ptr(flat), ptr(plan_src.pos), ptr(plan_src.offsets),
                                        ptr(wf), c_int(t), c_int(k), c_int(self.hidden), c_int(self.e_local),
                                        c_int(self.cap_rows), ptr(self.my_base), self._slab_ptrs, c_int(self.me),
                                        c_int(self.ep), ptr(counts_l), ptr(offsets_l), ptr(slot_rank), ptr(slot_row), st),
              "moe_p2p_dispatch")
        self.arena.barrier(self.ranks)
        self.calls += 1
        plan = K.MoePlan(counts_l, offsets_l, None, tiles, self.cap_rows, 0, 1, self.e_local)
        return Route(plan, slot_rank, slot_row, t, k)

    def combine(self, route: Route, weights: Optional[torch.Tensor], keep_rows: bool = False
                ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """``out[t] = sum_j weights[t, j] * out_slab_of(rank(t, j))[row(t, j)]``; ``keep_rows`` also returns
        the pulled rows ``[T*k, H]`` (what the gradient of the weights needs)."""
        self.arena.barrier(self.ranks)                             # every rank's expert outputs are in its out_slab
        dev = self.slab.device
        out = guard.empty(route.tokens, self.hidden, dtype=self.slab.dtype, device=dev)
        rows = guard.empty(route.tokens * route.k, self.hidden, dtype=self.slab.dtype, device=dev) if keep_rows else None
        wf = None if weights is None else weights.reshape(-1).float().contiguous()
        check(self.arena.lib.msrl_moe_p2p_combine(self._out_ptrs, c_int(self.ep), ptr(route.slot_rank),
                                                  ptr(route.slot_row), ptr(wf), c_int(route.tokens), c_int(route.k),
                                                  c_int(self.hidden), c_int(self.cap_rows), ptr(out), c_ll(self.hidden),
                                                  ptr(rows), stream()), "moe_p2p_combine")
        return out, rows


_dispatchers = {}


def dispatcher_for(arena: Optional[SymmetricArena], ep_group, experts_local: int, hidden: int, cap_rows: int,
                   dtype: torch.dtype, fallback: bool = True) -> Optional[P2PDispatcher]:
    """The shared dispatcher of this expert-parallel group, created on first use (every member
    reaches this call at the same point, so the arena offsets agree); ``None`` when the buffers do
    not fit or the shapes are outside the kernels' cover."""
    if arena is None or cap_rows <= 0 or dtype != torch.bfloat16 or hidden % 8:
        return None
    key = (id(arena), id(ep_group), experts_local, hidden, cap_rows)
    if key not in _dispatchers:
        ranks = arena.team_ranks(ep_group)
        need = P2PDispatcher.bytes_needed(len(ranks), experts_local, hidden, cap_rows)
        _dispatchers[key] = P2PDispatcher(arena, ranks, experts_local, hidden, cap_rows, dtype, fallback=fallback) \
            if arena.free_bytes() >= need else None
    return _dispatchers[key]
