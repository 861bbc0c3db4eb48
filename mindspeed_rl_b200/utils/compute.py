"""Token log-probabilities, entropy and KL penalties.

* ``compute_kl_penalty`` -- the four estimators ``kl | abs | mse | low_var_kl`` with the
  reference's clamps (``mindspeed_rl/utils/compute.py:100-133``).
* ``vocab_parallel_log_probs`` / ``vocab_parallel_entropy`` -- the un-fused formulation over a
  vocabulary that is sharded across a tensor-parallel group: three all-reduces (max,
  sum-exp, target logit / sum p*z).  This is the NCCL baseline path and the autograd oracle
  for the fused LM-head kernel in ``ops.lmhead_logprob`` (reference call sites:
  ``utils/compute.py:29-97``).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist


def compute_kl_penalty(logprob: torch.Tensor, ref_logprob: torch.Tensor,
                       kl_penalty: str = "kl") -> torch.Tensor:
    if kl_penalty == "kl":
        return logprob - ref_logprob
    if kl_penalty == "abs":
        return (logprob - ref_logprob).abs()
    if kl_penalty == "mse":
        return 0.5 * (logprob - ref_logprob).square()
    if kl_penalty == "low_var_kl":
        # k3 estimator: e^k - k - 1 with k = ref - logp, both clamped for stability
        k = torch.clamp(ref_logprob - logprob, min=-20.0, max=20.0)
        return torch.clamp(torch.exp(k) - k - 1.0, min=-10.0, max=10.0)
    raise NotImplementedError(f"unknown kl_penalty '{kl_penalty}'")


def _group_size(group) -> int:
    if group is None or not dist.is_available() or not dist.is_initialized():
        return 1
    return dist.get_world_size(group)


def _vocab_range(partition: int, group) -> Tuple[int, int]:
    if _group_size(group) == 1:
        return 0, partition
    r = dist.get_rank(group)
    return r * partition, (r + 1) * partition


class _VocabParallelLogProb(torch.autograd.Function):
    """log p(target) over logits sharded on the last dim across ``group``."""

    @staticmethod
    def forward(ctx, logits: torch.Tensor, target: torch.Tensor, group):
        z = logits.float()
        part = z.size(-1)
        lo, hi = _vocab_range(part, group)
        zmax = z.max(dim=-1).values
        multi = _group_size(group) > 1
        if multi:
            dist.all_reduce(zmax, op=dist.ReduceOp.MAX, group=group)
        z = z - zmax.unsqueeze(-1)
        mine = (target >= lo) & (target < hi)
        local_t = torch.where(mine, target - lo, torch.zeros_like(target))
        tgt = z.gather(-1, local_t.unsqueeze(-1)).squeeze(-1)
        tgt = torch.where(mine, tgt, torch.zeros_like(tgt))
        ez = z.exp()
        denom = ez.sum(dim=-1)
        if multi:
            dist.all_reduce(tgt, group=group)
            dist.all_reduce(denom, group=group)
        ctx.save_for_backward(ez / denom.unsqueeze(-1), mine, local_t)
        ctx.in_dtype = logits.dtype
        return tgt - denom.log()

    @staticmethod
    def backward(ctx, grad_out):
        probs, mine, local_t = ctx.saved_tensors
        grad = -probs
        one = mine.to(grad.dtype).unsqueeze(-1)
        grad.scatter_add_(-1, local_t.unsqueeze(-1), one)
        grad = grad * grad_out.unsqueeze(-1)
        return grad.to(ctx.in_dtype), None, None


def vocab_parallel_log_probs(logits: torch.Tensor, labels: torch.Tensor,
                             group=None) -> torch.Tensor:
    """Per-token ``log softmax(logits)[labels]`` for vocab-sharded ``logits``."""
    return _VocabParallelLogProb.apply(logits, labels, group)


def compute_log_probs(logits: torch.Tensor, labels: torch.Tensor, group=None, **_) -> torch.Tensor:
    """Name kept for callers that used the reference helper (``utils/compute.py:29-51``)."""
    return vocab_parallel_log_probs(logits, labels, group)


class _VocabParallelEntropy(torch.autograd.Function):
    """H = max + log sum e^(z-max) - sum softmax*z over a sharded vocabulary."""

    @staticmethod
    def forward(ctx, logits: torch.Tensor, group):
        z = logits.float()
        multi = _group_size(group) > 1
        zmax = z.max(dim=-1, keepdim=True).values
        if multi:
            dist.all_reduce(zmax, op=dist.ReduceOp.MAX, group=group)
        ez = (z - zmax).exp()
        denom = ez.sum(dim=-1, keepdim=True)
        if multi:
            dist.all_reduce(denom, group=group)
        p = ez / denom
        pz = (p * z).sum(dim=-1, keepdim=True)
        if multi:
            dist.all_reduce(pz, group=group)
        ctx.save_for_backward(z, p, pz)
        ctx.in_dtype = logits.dtype
        return (zmax + denom.log() - pz).squeeze(-1)

    @staticmethod
    def backward(ctx, grad_out):
        z, p, pz = ctx.saved_tensors
        # dH/dz_j = p_j * (sum_k p_k z_k - z_j)
        grad = p * (pz - z) * grad_out.unsqueeze(-1)
        return grad.to(ctx.in_dtype), None


def vocab_parallel_entropy(logits: torch.Tensor, group=None) -> torch.Tensor:
    return _VocabParallelEntropy.apply(logits, group)


def log_probs_and_entropy(logits: torch.Tensor, labels: torch.Tensor, group=None,
                          want_entropy: bool = True) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    lp = vocab_parallel_log_probs(logits, labels, group)
    ent = vocab_parallel_entropy(logits, group) if want_entropy else None
    return lp, ent
