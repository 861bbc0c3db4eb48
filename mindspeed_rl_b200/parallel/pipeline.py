"""Pipeline-parallel schedules over point-to-point exchanges of packed activations.

Every pipeline stage holds a slice of the decoder (``GPTModel(pre_process=..., post_process=...,
layer_numbers=...)``); all stages of a model replica receive the same micro-batches, so the shape
of every activation that crosses a stage boundary (``[tokens / sp, hidden]``) is known on both
sides and no shape handshake is needed.

* ``forward_only``: micro-batches stream through the stages; the last stage returns the outputs.
* ``forward_backward`` (non-interleaved 1F1B): ``pp - rank - 1`` warm-up forwards, then one
  forward / one backward in steady state, then the cool-down backwards -- at most ``pp - rank``
  micro-batches of activations are alive on a stage.  Sends and receives that could face each
  other are issued together (``batch_isend_irecv``) so neighbouring stages never block on each
  other.

Role in the reference: Megatron's ``get_forward_backward_func()`` schedules, called from
``mindspeed_rl/models/base/base_training_engine.py:189-279``.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


class PipelineSchedule:
    def __init__(self, group, rank: int, size: int, prev_rank: int, next_rank: int, hidden_size: int,
                 dtype: torch.dtype, device, seq_shard: int = 1):
        """``prev_rank`` / ``next_rank`` are global ranks; ``seq_shard`` is the TP size when
        sequence parallelism shards activations over tokens (else 1)."""
        self.group, self.rank, self.size = group, rank, size
        self.prev_rank, self.next_rank = prev_rank, next_rank
        self.hidden_size, self.dtype, self.device = hidden_size, dtype, torch.device(device)
        self.seq_shard = seq_shard

    @property
    def is_first(self) -> bool:
        return self.rank == 0

    @property
    def is_last(self) -> bool:
        return self.rank == self.size - 1

    # ---- p2p -------------------------------------------------------------------------------------
    def _buf(self, tokens: int) -> torch.Tensor:
        return torch.empty(tokens // self.seq_shard, self.hidden_size, dtype=self.dtype, device=self.device)

    def _exchange(self, send_next=None, send_prev=None, recv_prev_tokens: Optional[int] = None,
                  recv_next_tokens: Optional[int] = None) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
        ops, from_prev, from_next = [], None, None
        if send_prev is not None:
            ops.append(dist.P2POp(dist.isend, send_prev.contiguous(), self.prev_rank, self.group))
        if recv_prev_tokens is not None:
            from_prev = self._buf(recv_prev_tokens)
            ops.append(dist.P2POp(dist.irecv, from_prev, self.prev_rank, self.group))
        if send_next is not None:
            ops.append(dist.P2POp(dist.isend, send_next.contiguous(), self.next_rank, self.group))
        if recv_next_tokens is not None:
            from_next = self._buf(recv_next_tokens)
            ops.append(dist.P2POp(dist.irecv, from_next, self.next_rank, self.group))
        if ops:
            for req in dist.batch_isend_irecv(ops):
                req.wait()
        return from_prev, from_next

    # ---- schedules ---------------------------------------------------------------------------------
    def forward_only(self, micro_batches: Sequence[Any], tokens_of: Callable[[Any], int],
                     stage_forward: Callable[[Any, Optional[torch.Tensor]], Any]) -> List[Any]:
        """``stage_forward(mb, h_in)`` returns hidden states (inner stages) or the stage outputs
        (last stage).  Returns the last stage's outputs (empty list elsewhere)."""
        outs = []
        for mb in micro_batches:
            h_in = None if self.is_first else self._exchange(recv_prev_tokens=tokens_of(mb))[0]
            out = stage_forward(mb, h_in)
            if self.is_last:
                outs.append(out)
            else:
                self._exchange(send_next=out)
        return outs

    def forward_backward(self, micro_batches: Sequence[Any], tokens_of: Callable[[Any], int],
                         stage_forward: Callable[[Any, Optional[torch.Tensor]], Any],
                         last_stage_backward: Callable[[Any, Any], Any]) -> List[Any]:
        """1F1B.  ``stage_forward(mb, h_in)`` must return an autograd-connected tensor (inner
        stages) or whatever ``last_stage_backward(mb, out)`` consumes (last stage; it runs the loss
        and ``backward`` itself and returns per-micro-batch statistics).  Returns those
        statistics on the last stage."""
        n = len(micro_batches)
        warm = min(self.size - self.rank - 1, n)
        pending: List[Tuple[Any, Optional[torch.Tensor], Any]] = []   # (mb, h_in, out) awaiting backward
        stats: List[Any] = []

        def fwd(i: int, h_in: Optional[torch.Tensor]):
            mb = micro_batches[i]
            if h_in is not None:
                h_in.requires_grad_(True)
            out = stage_forward(mb, h_in)
            pending.append((mb, h_in, out))
            return out

        def bwd(d_out: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
            mb, h_in, out = pending.pop(0)
            if self.is_last:
                stats.append(last_stage_backward(mb, out))
            else:
                torch.autograd.backward(out, d_out)
            return None if h_in is None else h_in.grad

        def recv_fwd(i: int) -> Optional[torch.Tensor]:
            return None if self.is_first else self._exchange(recv_prev_tokens=tokens_of(micro_batches[i]))[0]

        # warm-up forwards
        for i in range(warm):
            out = fwd(i, recv_fwd(i))
            self._exchange(send_next=out.detach())
        remaining = n - warm
        h_in = recv_fwd(warm) if remaining > 0 else None
        # steady state: forward micro-batch warm+k, backward micro-batch k
        for k in range(remaining):
            out = fwd(warm + k, h_in)
            if self.is_last:
                d_out = None
            else:
                d_out = self._exchange(send_next=out.detach(),
                                       recv_next_tokens=tokens_of(pending[0][0]))[1]
            d_in = bwd(d_out)
            more = k + 1 < remaining
            if self.is_first:
                h_in = None
            else:
                h_in = self._exchange(send_prev=d_in, recv_prev_tokens=tokens_of(micro_batches[warm + k + 1])
                                      if more else None)[0]
        # cool-down backwards
        for _ in range(warm):
            d_out = self._exchange(recv_next_tokens=tokens_of(pending[0][0]))[1]
            d_in = bwd(d_out)
            if not self.is_first:
                self._exchange(send_prev=d_in)
        return stats
