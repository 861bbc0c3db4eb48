"""Inference forward of the rollout engine over a paged KV cache.

The runner owns no parameters: ``RolloutWeights`` is a set of tensors (views into the reshard
arena, or aliases of the training parameters when the layouts coincide) re-bound before every
rollout phase (reference contract: ``VLLMInferEngine.sync_model_weights``,
``mindspeed_rl/models/rollout/vllm_engine.py:381-405``).

Two entry points: ``prefill`` (packed prompt chunks, varlen attention, KV written to the cache)
and ``decode`` (one token per sequence, paged attention).  Decode steps are replayed from CUDA
graphs captured per batch-size bucket; all graph inputs live in static buffers.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from .. import ops
from ..models.transformer_config import TransformerConfig
from ..ops import QKVLayout
from ..ops.gemm import linear_fwd
from ..parallel.tp_comm import NO_TP, TPComm


@dataclass
class LayerWeights:
    input_norm: torch.Tensor
    qkv_w: torch.Tensor
    qkv_b: Optional[torch.Tensor]
    o_w: torch.Tensor
    post_norm: torch.Tensor
    gate_up_w: Optional[torch.Tensor] = None
    down_w: Optional[torch.Tensor] = None
    q_norm: Optional[torch.Tensor] = None
    k_norm: Optional[torch.Tensor] = None
    moe: Optional[object] = None      # rollout.moe.MoEWeights for expert layers
    mla: Optional[object] = None      # models.mla.MLASelfAttention of a latent-attention layer (replaces qkv_w)


@dataclass
class RolloutWeights:
    embed: torch.Tensor
    layers: List[LayerWeights]
    final_norm: torch.Tensor
    lm_head: torch.Tensor
    qkv_layout: QKVLayout
    vocab_start: int = 0


class KVCache:
    def __init__(self, num_layers: int, num_blocks: int, block_size: int, nkv: int, hd: int,
                 dtype, device):
        shape = (num_layers, num_blocks, block_size, nkv, hd)
        # uninitialised on the GPU: a slot is always written before any attention reads it, and
        # zero-filling tens of GB costs ~10 ms per rollout phase.  (The CPU reference path
        # gathers whole blocks, so it keeps the zero fill.)
        alloc = torch.empty if torch.device(device).type == "cuda" else torch.zeros
        self.k = alloc(shape, dtype=dtype, device=device)
        self.v = alloc(shape, dtype=dtype, device=device)
        self.num_blocks, self.block_size = num_blocks, block_size

    @staticmethod
    def bytes_per_block(num_layers, block_size, nkv, hd, dtype) -> int:
        return 2 * num_layers * block_size * nkv * hd * torch.empty(0, dtype=dtype).element_size()

    def copy_block(self, src: int, dst: int) -> None:
        self.k[:, dst].copy_(self.k[:, src])
        self.v[:, dst].copy_(self.v[:, src])


class ModelRunner:
    def __init__(self, cfg: TransformerConfig, device, comm: Optional[TPComm] = None,
                 max_model_len: int = 4096, enforce_eager: bool = True,
                 graph_batch_sizes: Tuple[int, ...] = ()):
        self.cfg = cfg
        self.device = torch.device(device)
        self.comm = comm or NO_TP
        self.max_model_len = max_model_len
        self.enforce_eager = enforce_eager or self.device.type != "cuda"
        self.graph_batch_sizes = tuple(sorted(graph_batch_sizes))
        self.weights: Optional[RolloutWeights] = None
        self.cache: Optional[KVCache] = None
        self._rope = None
        self._graphs: Dict[tuple, dict] = {}
        self._static: Optional[dict] = None
        self.prefix_tile = 0      # key tile of the tcgen05 shared-prefix kernel (set by the engine; 0 = mma.sync kernel)

    # ------------------------------------------------------------------------------------------
    def bind_weights(self, weights: Optional[RolloutWeights]) -> None:
        """(Re)bind parameters; graphs stay valid as long as the tensors keep their addresses."""
        old = self.weights
        self.weights = weights
        if weights is None or old is None or self._signature(old) != self._signature(weights):
            self._graphs.clear()

    @staticmethod
    def _signature(w: RolloutWeights):
        return (w.embed.data_ptr(), w.lm_head.data_ptr(), tuple((l.qkv_w if l.qkv_w is not None else l.o_w).data_ptr() for l in w.layers))

    def bind_cache(self, cache: Optional[KVCache]) -> None:
        self.cache = cache
        self._graphs.clear()
        self._static = None

    def rope_table(self) -> torch.Tensor:
        if self._rope is None:
            c = self.cfg
            self._rope = ops.rope_table(max(c.max_position_embeddings, self.max_model_len), c.head_dim,
                                        c.rotary_base, self.device, c.rope_scaling)
        return self._rope

    # ------------------------------------------------------------------------------------------
    def _embed(self, ids: torch.Tensor) -> torch.Tensor:
        w = self.weights
        if self.comm.world_size == 1:
            return w.embed[ids]
        local = ids - w.vocab_start
        mine = (local >= 0) & (local < w.embed.shape[0])
        h = w.embed[local.clamp(0, w.embed.shape[0] - 1)] * mine.unsqueeze(-1).to(w.embed.dtype)
        return self.comm.all_reduce(h)

    def _layer(self, li: int, lw: LayerWeights, resid, delta, positions, attend, rope_tab=None):
        cfg = self.cfg
        x, _, resid = ops.rmsnorm_fwd(delta, lw.input_norm, cfg.norm_epsilon, residual=resid,
                                      want_rstd=False) if resid is not None else \
            (*ops.rmsnorm_fwd(delta, lw.input_norm, cfg.norm_epsilon, want_rstd=False)[:2], delta)
        lay = self.weights.qkv_layout
        if lw.mla is not None:
            # latent attention: full per-head q / k / v (rotary and soft-max scale already applied)
            qkv = lw.mla.rollout_qkv(x, positions)
        else:
            qkv = linear_fwd(x, lw.qkv_w, lw.qkv_b)
            if lw.q_norm is not None:
                ops.headnorm_fwd_(qkv, lay, "q", lw.q_norm, cfg.norm_epsilon)
                ops.headnorm_fwd_(qkv, lay, "k", lw.k_norm, cfg.norm_epsilon)
            ops.rope_(qkv, lay, positions, self.rope_table() if rope_tab is None else rope_tab)
        attn = attend(li, qkv, lay)
        delta = self.comm.all_reduce(linear_fwd(attn, lw.o_w))
        x, _, resid = ops.rmsnorm_fwd(delta, lw.post_norm, cfg.norm_epsilon, residual=resid,
                                      want_rstd=False)
        if lw.moe is not None:
            delta = lw.moe.forward(x, self.comm)
        else:
            y = ops.swiglu_fwd(linear_fwd(x, lw.gate_up_w))
            delta = self.comm.all_reduce(linear_fwd(y, lw.down_w))
        return resid, delta

    @torch.no_grad()
    def idle_forward(self) -> None:
        """The collective part of a forward for a rank that has no tokens this step: every expert
        layer joins its group's token exchange with zero tokens (and serves the other ranks' tokens
        that are routed to its experts)."""
        empty = torch.zeros(0, self.cfg.hidden_size, dtype=self.cfg.params_dtype, device=self.device)
        for lw in self.weights.layers:
            if lw.moe is not None:
                lw.moe.forward(empty, self.comm)

    def _forward(self, ids, positions, attend, mm: Optional[dict] = None) -> torch.Tensor:
        """Returns the final hidden states ``[T, H]`` (after the last norm).  ``mm`` (vision-language
        prompts): ``image_index`` / ``image_embeds`` replace placeholder embeddings, ``rope_table [T, d]``
        is the per-token rotary table of three-axis positions (``positions`` then numbers the tokens)."""
        w = self.weights
        resid, delta = None, self._embed(ids)
        rope_tab = None
        if mm is not None:
            if mm.get("image_index") is not None and mm["image_index"].numel():
                delta = delta.index_copy(0, mm["image_index"], mm["image_embeds"].to(delta.dtype))
            rope_tab = mm.get("rope_table")
        for li, lw in enumerate(w.layers):
            resid, delta = self._layer(li, lw, resid, delta, positions, attend, rope_tab)
        x, _, _ = ops.rmsnorm_fwd(delta, w.final_norm, self.cfg.norm_epsilon, residual=resid,
                                  want_rstd=False)
        return x

    def _logits(self, x: torch.Tensor) -> torch.Tensor:
        return linear_fwd(x, self.weights.lm_head)

    # ------------------------------------------------------------------------------------------
    @torch.no_grad()
    def prefill(self, ids: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor,
                cu_q: torch.Tensor, max_q: int, last_index: torch.Tensor,
                prefix: Optional[dict] = None, mm: Optional[dict] = None) -> torch.Tensor:
        """Run packed prompt chunks. ``last_index`` selects the rows whose logits are needed.

        ``prefix`` (for chunks that start inside a sequence) carries ``block_tables``,
        ``token_seq``, ``token_pos``, ``cu_k``: the K/V of ``[0, chunk_end)`` is gathered from the
        cache after this chunk's K/V has been written.
        """
        cache = self.cache

        def attend(li, qkv, lay):
            ops.kv_cache_write(qkv, lay, slots, cache.k[li], cache.v[li])
            if prefix is None:
                out, _ = ops.attn_varlen_fwd(qkv, lay, cu_q, max_q, causal=True)
                return out
            k, v = ops.kv_cache_gather(cache.k[li], cache.v[li], prefix["block_tables"],
                                       prefix["token_seq"], prefix["token_pos"])
            out, _ = ops.attn_varlen_fwd(qkv, lay, cu_q, max_q, causal=True, kv=(k, v),
                                         cu_seqlens_k=prefix["cu_k"])
            return out

        x = self._forward(ids, positions, attend, mm)
        return self._logits(x[last_index])

    # ------------------------------------------------------------------------------------------
    def _decode_eager(self, ids, positions, slots, block_tables, context_lens, max_context, groups=None):
        cache = self.cache

        def attend(li, qkv, lay):
            ops.kv_cache_write(qkv, lay, slots, cache.k[li], cache.v[li])
            return ops.paged_decode_attention(qkv, lay, cache.k[li], cache.v[li], block_tables,
                                              context_lens, max_context, groups=groups,
                                              prefix_tile=self.prefix_tile if groups is not None else 0)

        return self._logits(self._forward(ids, positions, attend))

    def _ensure_static(self, max_blocks: int) -> dict:
        cap = self.graph_batch_sizes[-1]
        st = self._static
        if st is None or st["block_tables"].shape[1] < max_blocks:
            dev = self.device
            st = dict(ids=torch.zeros(cap, dtype=torch.int64, device=dev),
                      positions=torch.zeros(cap, dtype=torch.int32, device=dev),
                      slots=torch.full((cap,), -1, dtype=torch.int64, device=dev),
                      block_tables=torch.zeros(cap, max_blocks, dtype=torch.int32, device=dev),
                      context_lens=torch.zeros(cap, dtype=torch.int32, device=dev),
                      key_start=torch.zeros(cap, dtype=torch.int32, device=dev),
                      group_rows=torch.full((cap, 8), -1, dtype=torch.int32, device=dev),
                      group_prefix=torch.zeros(cap, dtype=torch.int32, device=dev))
            self._static = st
            self._graphs.clear()
        return st

    @torch.no_grad()
    def decode(self, ids: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor,
               block_tables: torch.Tensor, context_lens: torch.Tensor, max_context: int,
               groups=None) -> torch.Tensor:
        """One token per sequence -> logits ``[B, V_local]``.  ``groups`` (see
        ``ops.paged_decode_attention``; an optional fourth entry gives the number of groups that have
        members, which come first in the tables) turns on shared-prefix attention for n-sample groups.
        Shared prefixes must be multiples of ``self.prefix_tile`` keys when that is non-zero."""
        b = ids.shape[0]
        bucket = next((s for s in self.graph_batch_sizes if s >= b), None)
        n_groups = b
        if groups is not None:
            if len(groups) > 3:
                # the shared pass launches one CTA per listed group: list a power of two that covers the real ones
                n_groups = min(b, 1 << max(0, int(groups[3]) - 1).bit_length())
            groups = tuple(groups[:3])
        if self.enforce_eager or bucket is None:
            if groups is not None:
                groups = (groups[0], groups[1][:n_groups], groups[2][:n_groups])
            return self._decode_eager(ids, positions, slots, block_tables, context_lens, max_context, groups)
        max_blocks = (self.max_model_len + self.cache.block_size - 1) // self.cache.block_size
        st = self._ensure_static(max_blocks)
        st["ids"][:b].copy_(ids)
        st["positions"][:b].copy_(positions)
        st["slots"][:b].copy_(slots)
        st["slots"][b:bucket].fill_(-1)
        st["context_lens"][:b].copy_(context_lens)
        st["context_lens"][b:bucket].zero_()
        st["block_tables"][:b, :block_tables.shape[1]].copy_(block_tables)
        grouped = groups is not None
        if grouped:
            st["key_start"][:b].copy_(groups[0])
            st["key_start"][b:bucket].zero_()
            st["group_rows"][:b].copy_(groups[1])
            st["group_rows"][b:bucket].fill_(-1)
            st["group_prefix"][:b].copy_(groups[2])
        n_groups = min(n_groups, bucket) if grouped else 0
        g = self._graphs.get((bucket, grouped, n_groups))
        if g is None:
            g = self._capture(bucket, st, grouped, n_groups)
        g["graph"].replay()
        return g["logits"][:b]

    def _capture(self, bucket: int, st: dict, grouped: bool = False, n_groups: int = 0) -> dict:
        groups = (st["key_start"][:bucket], st["group_rows"][:n_groups], st["group_prefix"][:n_groups]) if grouped else None
        args = (st["ids"][:bucket], st["positions"][:bucket], st["slots"][:bucket],
                st["block_tables"][:bucket], st["context_lens"][:bucket], self.max_model_len, groups)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):       # warm-up: sizes scratch buffers outside the capture
            self._decode_eager(*args)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            logits = self._decode_eager(*args)
        rec = dict(graph=graph, logits=logits)
        self._graphs[(bucket, grouped, n_groups)] = rec
        return rec
