"""Pipeline-parallel schedules over point-to-point exchanges of packed activations.

Every pipeline stage holds a slice of the decoder (``GPTModel(pre_process=..., post_process=...,
layer_numbers=...)``); all stages of a model replica receive the same micro-batches, so the shape
of every activation that crosses a stage boundary (``[tokens / sp, hidden]``) is known on both
sides and no shape handshake is needed.

With ``num_chunks`` > 1 every rank holds several model chunks (virtual pipeline stages: chunk ``c``
of rank ``r`` is virtual stage ``c * pp + r``) and a micro-batch goes round the ring of ranks once
per chunk; activations travel on the pipeline group, gradients on a second group over the same
ranks, so that with two ranks (next == previous) a tensor can never be taken for the other kind.

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
                 dtype: torch.dtype, device, seq_shard: int = 1, num_chunks: int = 1, grad_group=None):
        """``prev_rank`` / ``next_rank`` are global ranks; ``seq_shard`` is the TP size when
        sequence parallelism shards activations over tokens (else 1); ``num_chunks``: model chunks
        per rank (interleaved schedule), ``grad_group``: second group over the same ranks."""
        self.group, self.rank, self.size = group, rank, size
        self.num_chunks = num_chunks
        self.grad_group = grad_group if grad_group is not None else group
        if num_chunks > 1 and grad_group is None:
            raise ValueError("the interleaved schedule needs a second process group for gradients")
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

    def _ring(self, group, send=None, send_to: Optional[int] = None, recv_tokens: Optional[int] = None,
              recv_from: Optional[int] = None) -> Optional[torch.Tensor]:
        """One batched send / receive on ``group`` (either part may be absent)."""
        ops, got = [], None
        if send is not None:
            ops.append(dist.P2POp(dist.isend, send.contiguous(), send_to, group))
        if recv_tokens is not None:
            got = self._buf(recv_tokens)
            ops.append(dist.P2POp(dist.irecv, got, recv_from, group))
        if ops:
            for req in dist.batch_isend_irecv(ops):
                req.wait()
        return got

    # ---- interleaved (virtual stages) ----------------------------------------------------------------
    def _virtual(self, k: int, n: int, forward: bool) -> Tuple[int, int]:
        """``k``-th forward (or backward) of this rank -> ``(micro-batch index, chunk)``: groups of
        ``pp`` micro-batches go through chunk 0, then chunk 1, ... (backward: chunks in reverse)."""
        p, v = self.size, self.num_chunks
        g, rem = divmod(k, p * v)
        c = rem // p
        return g * p + rem % p, (c if forward else v - 1 - c)

    def _first_virtual(self, chunk: int) -> bool:
        return self.rank == 0 and chunk == 0

    def _last_virtual(self, chunk: int) -> bool:
        return self.rank == self.size - 1 and chunk == self.num_chunks - 1

    def forward_only_interleaved(self, micro_batches, tokens_of, stage_forward) -> List[Any]:
        """Chunk by chunk: all micro-batches stream through chunk 0 of all ranks, then chunk 1, ...
        The outputs of the last rank for the next chunk of the first rank wait in flight on the
        second group, so the ring never blocks the pipeline of the current chunk."""
        outs, wrap_sends = [], []
        for c in range(self.num_chunks):
            for mb in micro_batches:
                if self._first_virtual(c):
                    h_in = None
                elif self.rank == 0:
                    h_in = self._buf(tokens_of(mb))
                    dist.recv(h_in, self.prev_rank, group=self.grad_group)
                else:
                    h_in = self._exchange(recv_prev_tokens=tokens_of(mb))[0]
                out = stage_forward(mb, h_in, c)
                if self._last_virtual(c):
                    outs.append(out)
                elif self.rank == self.size - 1:
                    t = out.contiguous()
                    wrap_sends.append((dist.isend(t, self.next_rank, group=self.grad_group), t))
                else:
                    self._exchange(send_next=out)
        for req, _ in wrap_sends:
            req.wait()
        return outs

    def forward_backward_interleaved(self, micro_batches, tokens_of, stage_forward, last_stage_backward) -> List[Any]:
        """Interleaved 1F1B over virtual stages (the schedule of Megatron's
        ``forward_backward_pipelining_with_interleaving``): ``(pp - rank - 1) * 2 + (chunks - 1) * pp``
        warm-up forwards, then one forward / one backward per step with one four-way exchange
        (activation to the next rank, gradient to the previous one, next inputs from both sides),
        then the cool-down backwards.  ``stage_forward(mb, h_in, chunk)``; the number of micro-batches
        must be a multiple of the pipeline size."""
        p, v, r = self.size, self.num_chunks, self.rank
        n = len(micro_batches)
        if n % p:
            raise ValueError(f"the interleaved schedule needs a multiple of {p} micro-batches, got {n}")
        total = n * v
        warm = total if n == p else min((p - r - 1) * 2 + (v - 1) * p, total)
        remaining = total - warm
        all_warmup = remaining == 0
        inputs: List[List[Optional[torch.Tensor]]] = [[] for _ in range(v)]     # received activations per chunk
        grads: List[List[Optional[torch.Tensor]]] = [[] for _ in range(v)]      # received output gradients per chunk
        pending: List[List[Tuple[Any, Optional[torch.Tensor], Any]]] = [[] for _ in range(v)]
        stats: List[Any] = []
        fwd = lambda k: self._virtual(k, n, True)
        bwd = lambda k: self._virtual(k, n, False)

        def forward_step(k: int):
            i, c = fwd(k)
            h_in = None if self._first_virtual(c) else inputs[c].pop(0)
            if h_in is not None:
                h_in.requires_grad_(True)
            out = stage_forward(micro_batches[i], h_in, c)
            pending[c].append((micro_batches[i], h_in, out))
            return None if self._last_virtual(c) else out.detach()

        def backward_step(k: int):
            i, c = bwd(k)
            mb, h_in, out = pending[c].pop(0)
            if self._last_virtual(c):
                stats.append(last_stage_backward(mb, out))
            else:
                torch.autograd.backward(out, grads[c].pop(0))
            return None if (h_in is None or self._first_virtual(c)) else h_in.grad

        def exchange(out, d_in, next_fwd: Optional[int], next_bwd: Optional[int]) -> None:
            """Send what this step produced; receive the input of forward ``next_fwd`` and the output
            gradient of backward ``next_bwd`` (``None``: nothing to receive)."""
            if next_fwd is not None:
                i, c = fwd(next_fwd)
                got = self._ring(self.group, out, self.next_rank, tokens_of(micro_batches[i]), self.prev_rank)
                inputs[c].append(got)
            elif out is not None:
                self._ring(self.group, out, self.next_rank)
            if next_bwd is not None:
                i, c = bwd(next_bwd)
                got = self._ring(self.grad_group, d_in, self.prev_rank, tokens_of(micro_batches[i]), self.next_rank)
                grads[c].append(got)
            elif d_in is not None:
                self._ring(self.grad_group, d_in, self.prev_rank)

        def wants_input(k: int) -> bool:       # does forward k take its input from the previous rank?
            return k < total and not self._first_virtual(fwd(k)[1])

        def wants_grad(k: int) -> bool:        # does backward k take its gradient from the next rank?
            return k < total and not self._last_virtual(bwd(k)[1])

        if wants_input(0):
            exchange(None, None, 0, None)
        for k in range(warm):
            out = forward_step(k)
            first_grad = (k == warm - 1) and not all_warmup and wants_grad(0)
            exchange(out, None, k + 1 if wants_input(k + 1) else None, 0 if first_grad else None)
        for j in range(remaining):
            out = forward_step(warm + j)
            d_in = backward_step(j)
            more_fwd = j + 1 < remaining
            exchange(out, d_in, warm + j + 1 if (more_fwd and wants_input(warm + j + 1)) else None,
                     j + 1 if wants_grad(j + 1) else None)
        if all_warmup and wants_grad(0):
            exchange(None, None, None, 0)
        for k in range(remaining, total):
            d_in = backward_step(k)
            exchange(None, d_in, None, k + 1 if wants_grad(k + 1) else None)
        return stats

    # ---- schedules ---------------------------------------------------------------------------------
    def forward_only(self, micro_batches: Sequence[Any], tokens_of: Callable[[Any], int],
                     stage_forward: Callable[[Any, Optional[torch.Tensor]], Any]) -> List[Any]:
        """``stage_forward(mb, h_in)`` returns hidden states (inner stages) or the stage outputs
        (last stage).  Returns the last stage's outputs (empty list elsewhere)."""
        if self.num_chunks > 1:
            return self.forward_only_interleaved(micro_batches, tokens_of, stage_forward)
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
        if self.num_chunks > 1:
            return self.forward_backward_interleaved(micro_batches, tokens_of, stage_forward, last_stage_backward)
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
