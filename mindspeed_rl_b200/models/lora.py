"""Low-rank adapters (LoRA) on the linears of the transformer layer.

``y = x W^T + (alpha / r) (x A^T) B^T`` with ``A [r, in]`` (normal init) and ``B [out, r]`` (zero
init); the base weights are frozen, only ``A`` / ``B`` are trained (reference feature:
``docs/zh/features/grpo_lora.md``; the reference merges ``alpha/r * B A`` into the weights when it
reshards for rollout, ``workers/resharding/vllm_weight_container.py:336-420``).

Under tensor parallelism the adapter follows the base weight's split:

* column-parallel (``linear_qkv``, ``linear_fc1``): ``A`` replicated, ``B`` split over ``out``.  Each
  rank back-propagates only its output slice, so the tiny ``dy B`` ([tokens, r]) is all-reduced
  over TP inside ``column_bwd`` before ``A``'s gradient is formed.
* row-parallel (``linear_proj``, ``linear_fc2``): ``A`` split over ``in``, ``B`` replicated.  The tiny
  ``x A^T`` ([tokens, r]) is all-reduced over TP, after which every rank adds
  ``s * (xA^T)[its tokens] B^T`` to its (reduce-scattered or all-reduced) output; the big
  GEMM -> reduce-scatter stays one fused kernel.

``merged_weight`` gives ``W + s B A`` for the rollout engine; ``adapter_disabled`` turns the adapters
off so that the same backbone serves as the frozen reference policy.
"""
from __future__ import annotations

import contextlib
import math
from typing import Any, Dict, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

TARGETS = ("linear_qkv", "linear_proj", "linear_fc1", "linear_fc2")
_KIND = {"linear_qkv": "column", "linear_fc1": "column", "linear_proj": "row", "linear_fc2": "row"}


def attach(holder: nn.Module, name: str, cfg, device, gen, sequence_parallel: bool) -> None:
    """Give ``holder`` (a weight holder with ``.weight [out_local, in_local]``) adapter parameters."""
    r = cfg.lora_r
    out_l, in_l = holder.weight.shape
    dt = holder.weight.dtype
    a = torch.empty(r, in_l, dtype=torch.float32, device=device)
    a.normal_(0.0, 1.0 / math.sqrt(max(in_l, 1)), generator=gen)
    holder.lora_A = nn.Parameter(a.to(dt))
    holder.lora_B = nn.Parameter(torch.zeros(out_l, r, dtype=dt, device=device))
    holder.lora_scale = float(cfg.lora_alpha) / float(r)
    holder.lora_kind = _KIND[name]
    holder.lora_on = True
    holder.weight.requires_grad_(False)
    if getattr(holder, "bias", None) is not None:
        holder.bias.requires_grad_(False)
    tp = cfg.tensor_model_parallel_size
    if tp > 1:
        if holder.lora_kind == "column":
            holder.lora_A.tp_replicated = True           # its gradient is summed inside column_bwd
        else:
            holder.lora_B.tp_replicated = True
            holder.lora_B.tp_reduce_grad = bool(sequence_parallel)   # partial over the token shards


def active(holder) -> bool:
    return getattr(holder, "lora_A", None) is not None and holder.lora_on


def _accum(p: torch.Tensor, dy: torch.Tensor, x: torch.Tensor) -> None:
    g = getattr(p, "main_grad", None)
    if g is None:
        if p.grad is None:
            p.grad = torch.zeros_like(p)
        g = p.grad
    g.add_(torch.matmul(dy.t(), x).to(g.dtype))


# ---- column-parallel ---------------------------------------------------------------------------------
def column_fwd(holder, x_full: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """``y += s (x A^T) B_local^T``; returns ``x A^T`` for the backward."""
    xa = torch.matmul(x_full, holder.lora_A.t())
    y.addmm_(xa, holder.lora_B.t(), alpha=holder.lora_scale)
    return xa


def column_bwd(holder, x_full: torch.Tensor, xa: torch.Tensor, dy: torch.Tensor, comm) -> torch.Tensor:
    """Accumulates the adapter gradients; returns the extra input gradient for this rank's rows
    (token shard under SP, all tokens otherwise), to be added to the *reduced* ``dy W``.  Only the
    tiny ``dy B`` ([tokens, r]) is summed over TP, never a hidden-sized tensor."""
    s = holder.lora_scale
    _accum(holder.lora_B, dy * s, xa)
    dxa = torch.matmul(dy, holder.lora_B) * s
    if comm.world_size > 1:
        dist.all_reduce(dxa, group=comm.group)
    _accum(holder.lora_A, dxa, x_full)                     # complete (and identical) on every TP rank
    rows = dxa
    if comm.sequence_parallel:
        n = dxa.shape[0] // comm.world_size
        rows = dxa[comm.rank * n:(comm.rank + 1) * n]
    return torch.matmul(rows, holder.lora_A)


# ---- row-parallel --------------------------------------------------------------------------------------
def row_fwd(holder, a_local: torch.Tensor, out: torch.Tensor, comm) -> Tuple[torch.Tensor, torch.Tensor]:
    """``out`` is the already reduced output (token shard under SP, full otherwise); adds the
    adapter term in place and returns ``(sum over TP of a A^T, its rows matching out)``."""
    xa = torch.matmul(a_local, holder.lora_A.t())
    if comm.world_size > 1:
        dist.all_reduce(xa, group=comm.group)
    rows = xa
    if comm.sequence_parallel:
        n = xa.shape[0] // comm.world_size
        rows = xa[comm.rank * n:(comm.rank + 1) * n]
    out.addmm_(rows, holder.lora_B.t(), alpha=holder.lora_scale)
    return xa, rows


def row_bwd(holder, a_local: torch.Tensor, rows: torch.Tensor, dout: torch.Tensor, comm) -> torch.Tensor:
    """``dout``: gradient of the reduced output (token shard under SP).  Returns the extra
    gradient for ``a_local`` ``[tokens, in_local]``."""
    s = holder.lora_scale
    _accum(holder.lora_B, dout * s, rows)
    dxa = torch.matmul(dout, holder.lora_B) * s            # [tokens(/tp), r]
    if comm.sequence_parallel:
        full = torch.empty(dxa.shape[0] * comm.world_size, dxa.shape[1], dtype=dxa.dtype, device=dxa.device)
        dist.all_gather_into_tensor(full, dxa.contiguous(), group=comm.group)
        dxa = full
    _accum(holder.lora_A, dxa, a_local)
    return torch.matmul(dxa, holder.lora_A)


# ---- whole-model helpers ---------------------------------------------------------------------------------
def merged_weight(holder) -> torch.Tensor:
    """``W + s B A`` (new tensor) for an adapted holder, the plain weight otherwise."""
    if not active(holder):
        return holder.weight.data
    delta = torch.matmul(holder.lora_B.data.float(), holder.lora_A.data.float()) * holder.lora_scale
    return (holder.weight.data.float() + delta).to(holder.weight.dtype)


def holders(model: nn.Module):
    for m in model.modules():
        if getattr(m, "lora_A", None) is not None:
            yield m


@contextlib.contextmanager
def adapter_disabled(model: nn.Module):
    """Run the backbone without adapters (the frozen reference policy of LoRA training)."""
    hs = list(holders(model))
    old = [h.lora_on for h in hs]
    for h in hs:
        h.lora_on = False
    try:
        yield
    finally:
        for h, o in zip(hs, old):
            h.lora_on = o


def freeze_base(model: nn.Module) -> None:
    """Only adapter parameters stay trainable."""
    for n, p in model.named_parameters():
        if not (n.endswith("lora_A") or n.endswith("lora_B")):
            p.requires_grad_(False)
