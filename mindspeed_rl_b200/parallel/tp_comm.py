"""Tensor-parallel communication around the column / row linears of a transformer layer.

``TPComm`` hides which collective pattern a layer uses:

* plain TP: activations are replicated; row-parallel outputs are all-reduced;
* TP + sequence parallel: activations between layers are sharded over tokens; the
  column-parallel input is all-gathered and the row-parallel output reduce-scattered.

The NCCL implementation here is the baseline ("reference-equivalent") path; the fused
all-gather->GEMM and GEMM->reduce-scatter kernels plug in through ``fused_ag_gemm`` /
``fused_gemm_rs`` hooks when a symmetric-memory team is attached.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..ops.gemm import linear_dgrad, linear_fwd


class TPComm:
    def __init__(self, group=None, sequence_parallel: bool = False, world_size: Optional[int] = None,
                 rank: Optional[int] = None):
        self.group = group
        inited = dist.is_available() and dist.is_initialized()
        if world_size is None:
            world_size = dist.get_world_size(group) if (inited and group is not None) else 1
        if rank is None:
            rank = dist.get_rank(group) if (inited and group is not None) else 0
        self.world_size = world_size
        self.rank = rank
        self.sequence_parallel = sequence_parallel and world_size > 1
        self.fused = None  # optional object with ag_gemm / gemm_rs (parallel.fused_tp)
        self.peer_ar = None  # optional parallel.symm.PeerAllReduce for small bf16 messages (decode steps)

    # forward direction ---------------------------------------------------------------------------
    def gather_seq(self, x: torch.Tensor) -> torch.Tensor:
        """Before a column-parallel linear: all-gather tokens when sequence parallel."""
        if not self.sequence_parallel:
            return x
        out = torch.empty(x.shape[0] * self.world_size, *x.shape[1:], device=x.device, dtype=x.dtype)
        dist.all_gather_into_tensor(out, x.contiguous(), group=self.group)
        return out

    def reduce_out(self, y: torch.Tensor) -> torch.Tensor:
        """After a row-parallel linear: reduce-scatter (SP) or all-reduce partial sums."""
        if self.world_size == 1:
            return y
        if self.sequence_parallel:
            out = torch.empty(y.shape[0] // self.world_size, *y.shape[1:], device=y.device,
                              dtype=y.dtype)
            dist.reduce_scatter_tensor(out, y.contiguous(), group=self.group)
            return out
        return self.all_reduce(y)

    # backward direction (transposes of the above) -----------------------------------------------------
    def gather_seq_bwd(self, dx_full: torch.Tensor) -> torch.Tensor:
        """Gradient of :meth:`gather_seq`: reduce-scatter (SP) / all-reduce (input was replicated)."""
        return self.reduce_out(dx_full)

    def reduce_out_bwd(self, dy: torch.Tensor) -> torch.Tensor:
        """Gradient of :meth:`reduce_out`: all-gather (SP) / identity."""
        return self.gather_seq(dy)

    def all_reduce(self, t: torch.Tensor, op=None) -> torch.Tensor:
        if self.world_size > 1 and op is None and self.peer_ar is not None and self.peer_ar.fits(t):
            return self.peer_ar.all_reduce(t)      # one peer-memory kernel instead of a library collective
        if self.world_size > 1:
            dist.all_reduce(t, op=op or dist.ReduceOp.SUM, group=self.group)
        return t

    # linear + collective pairs ------------------------------------------------------------------------
    # With a symmetric-memory team attached (``self.fused``) and sequence parallelism on, each pair
    # runs as one communication-fused tcgen05 kernel; otherwise as collective + matmul.
    def _fused_ok(self, t: torch.Tensor) -> bool:
        return self.fused is not None and self.sequence_parallel and t.is_cuda

    def column_linear(self, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None):
        """``(gather_seq(x) @ w.T + bias, gather_seq(x))``."""
        if self._fused_ok(x) and self.fused.fits_ag(x, w):
            y, xg = self.fused.ag_gemm(x, w)
        else:
            xg = self.gather_seq(x)
            return linear_fwd(xg, w, bias), xg
        if bias is not None:
            y += bias
        return y, xg

    def row_linear(self, a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """``reduce_out(a @ w.T)``."""
        if self._fused_ok(a) and self.fused.fits_rs(a, w):
            return self.fused.gemm_rs(a, w)
        return self.reduce_out(linear_fwd(a, w))

    def column_linear_bwd(self, dy: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """Input gradient of :meth:`column_linear`: ``gather_seq_bwd(dy @ w)``."""
        if self._fused_ok(dy):
            wt = self.fused.transposed(w)
            if self.fused.fits_rs(dy, wt):
                return self.fused.gemm_rs(dy, wt)
        return self.gather_seq_bwd(linear_dgrad(dy, w))

    def row_linear_bwd(self, dout: torch.Tensor, w: torch.Tensor):
        """Input gradient of :meth:`row_linear`: ``(reduce_out_bwd(dout) @ w, reduce_out_bwd(dout))``
        (the gathered output gradient is what the weight gradient needs)."""
        if self._fused_ok(dout):
            wt = self.fused.transposed(w)
            if self.fused.fits_ag(dout, wt):
                return self.fused.ag_gemm(dout, wt)
        d_full = self.reduce_out_bwd(dout)
        return linear_dgrad(d_full, w), d_full


NO_TP = TPComm()
