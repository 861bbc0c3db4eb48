"""Communication-fused tensor-parallel linears over symmetric memory.

With sequence parallelism every column-parallel linear is "all-gather tokens, then GEMM" and
every row-parallel linear is "GEMM, then reduce-scatter tokens" (reference: Megatron
``ColumnParallelLinear`` / ``RowParallelLinear`` with ``sequence_parallel``, driven from
``mindspeed_rl/models/base/base_training_engine.py``).  ``FusedTP`` runs each pair as ONE
tcgen05 kernel (``csrc/gemm_tcgen05.cu``, variants COMM_AG / COMM_RS):

* ``ag_gemm``: the activation shard is written into a peer-mapped slot; after a device barrier
  the kernel's comm warps pull the peers' shards over NVLink into a local gathered buffer (each
  byte crosses once, and the gathered activations are kept for the weight gradient) while the
  tensor cores already multiply the tiles that have landed.
* ``gemm_rs``: the epilogue stores every partial tile straight into the owner rank's staging
  area and bumps its arrival counter; the owner's comm warps add the staged partials in fp32 as
  soon as a row tile is complete.  No barrier is needed: staging and counters are
  double-buffered by call parity, and a rank cannot run two calls ahead of a peer because its
  own reduction waits for that peer's tiles.

All ranks of the team must issue the same sequence of calls.  Shapes that do not fit (token
shard not a multiple of 128, operands not 16-byte aligned, buffers too small) fall back to the
library path of ``TPComm``.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional, Sequence, Tuple

import torch

from ..ops import _lib, guard
from ..ops.gemm import _ok_operand, _status_word
from ..ops._lib import c_int, c_ll

c_uint = ctypes.c_uint

_TILE = 128


class FusedTP:
    def __init__(self, arena, ranks: Sequence[int], max_local_tokens: int, max_k: int, max_n: int):
        """``ranks``: team positions of the tensor-parallel group inside ``arena``'s team;
        ``max_local_tokens``: largest token shard (rounded up to 128); ``max_k``: widest gathered
        activation (all-gather side); ``max_n``: widest reduced output (reduce-scatter side)."""
        self.arena = arena
        self.ranks = list(ranks)
        self.world = len(self.ranks)
        self.me = self.ranks.index(arena.rank)
        self.lib = _lib.load()
        import os
        self.use_pair = os.environ.get("MSRL_FUSED_TP_PAIR", "1") == "1"
        self.max_m = (max_local_tokens + _TILE - 1) // _TILE * _TILE
        self.max_k, self.max_n = max_k, max_n
        tiles = self.max_m // _TILE
        dev = arena.device
        # peer-visible buffers (same offsets on every rank of the team)
        self.x_slot = [arena.alloc((self.max_m, max_k), torch.bfloat16) for _ in range(2)]
        self.stage = [arena.alloc((self.world, self.max_m * max_n), torch.bfloat16) for _ in range(2)]
        self.flags = [arena.alloc(tiles, torch.int32).zero_() for _ in range(2)]
        # local scratch
        self.tile_ready = torch.zeros(self.world * tiles, dtype=torch.int32, device=dev)
        self.done = [torch.zeros(tiles, dtype=torch.int32, device=dev) for _ in range(2)]
        self._ag_calls = 0
        self._rs_calls = 0
        self._wt: Dict[int, Tuple[int, torch.Tensor]] = {}
        self.weights_epoch = 0
        torch.cuda.synchronize(dev)
        arena.barrier(self.ranks)            # buffers are zeroed everywhere before the first push

    # ------------------------------------------------------------------------------------------
    def fits_ag(self, x: torch.Tensor, w: torch.Tensor) -> bool:
        m, k = x.shape
        return (m % _TILE == 0 and 0 < m <= self.max_m and k <= self.max_k and k % 8 == 0
                and x.dtype == torch.bfloat16 and _ok_operand(w) and w.shape[1] == k)

    def fits_rs(self, a: torch.Tensor, w: torch.Tensor) -> bool:
        m, k = a.shape
        n = w.shape[0]
        ml = m // self.world
        return (m % (self.world * _TILE) == 0 and 0 < ml <= self.max_m and n <= self.max_n and n % 8 == 0
                and _ok_operand(a) and _ok_operand(w) and w.shape[1] == k)

    # ------------------------------------------------------------------------------------------
    def ag_gemm(self, x: torch.Tensor, w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """``x [m_local, K]`` (this rank's tokens), ``w [N, K]`` ->
        ``(all_gather(x) @ w.T  [world*m_local, N],  all_gather(x) [world*m_local, K])``."""
        ml, k = x.shape
        n = w.shape[0]
        slot = self.x_slot[self._ag_calls & 1].view(-1)[:ml * k].view(ml, k)
        self._ag_calls += 1
        slot.copy_(x)
        self.arena.barrier(self.ranks)       # every shard is in place (and the previous user of the other slot done)
        m = ml * self.world
        gathered = guard.empty(m, k, dtype=torch.bfloat16, device=x.device)
        out = guard.empty(m, n, dtype=torch.bfloat16, device=x.device)
        peers = self.arena.peer_ptrs(self.arena.offset_of(slot), self.ranks)
        # token shards in multiples of 256 rows run on CTA pairs (cta_group::2 main loop)
        fn = self.lib.msrl_ag_gemm_pair_bf16_tn if (ml % 256 == 0 and self.use_pair) else self.lib.msrl_ag_gemm_bf16_tn
        _lib.check(fn(
            peers, c_ll(k), _lib.ptr(gathered), _lib.ptr(w), c_ll(w.stride(0)), _lib.ptr(out), c_ll(n),
            c_int(ml), c_int(n), c_int(k), c_int(self.me), c_int(self.world), _lib.ptr(self.tile_ready),
            _lib.ptr(_status_word(x.device)), _lib.stream()), "ag_gemm")
        return out, gathered

    def gemm_rs(self, a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """``a [world*m_local, K_local]``, ``w [N, K_local]`` ->
        ``reduce_scatter(a @ w.T) [m_local, N]`` (this rank's token block)."""
        m, k = a.shape
        n = w.shape[0]
        ml = m // self.world
        par = self._rs_calls & 1
        self._rs_calls += 1
        out = guard.empty(ml, n, dtype=torch.bfloat16, device=a.device)
        stage_off = self.arena.offset_of(self.stage[par])
        flag_off = self.arena.offset_of(self.flags[par])
        tiles_n = int(self.lib.msrl_gemm_rs_tiles(c_int(n)))
        fn = self.lib.msrl_gemm_rs_pair_bf16_tn if (ml % 256 == 0 and self.use_pair) else self.lib.msrl_gemm_rs_bf16_tn
        _lib.check(fn(
            _lib.ptr(a), c_ll(a.stride(0)), _lib.ptr(w), c_ll(w.stride(0)),
            self.arena.peer_ptrs(stage_off, self.ranks), self.arena.peer_ptrs(flag_off, self.ranks),
            _lib.ptr(self.done[par]), _lib.ptr(out), c_ll(n), c_int(ml), c_int(n), c_int(k), c_int(self.me),
            c_int(self.world), c_uint(self.world * tiles_n * 4), _lib.ptr(_status_word(a.device)),
            _lib.stream()), "gemm_rs")
        return out

    # ------------------------------------------------------------------------------------------
    def transposed(self, w: torch.Tensor) -> torch.Tensor:
        """``w.T`` as a contiguous tensor, cached until ``weights_epoch`` moves (optimizer step):
        the backward data-gradient GEMMs ``dY @ W`` run through the same K-major kernels."""
        key = w.data_ptr()
        hit = self._wt.get(key)
        if hit is not None and hit[0] == self.weights_epoch and hit[1].shape == (w.shape[1], w.shape[0]):
            return hit[1]
        wt = w.t().contiguous()
        self._wt[key] = (self.weights_epoch, wt)
        return wt

    def invalidate_weights(self) -> None:
        self.weights_epoch += 1
