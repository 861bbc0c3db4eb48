"""Flat-buffer optimizer ops: sum of squares, device-side clip coefficient, fused AdamW.

CUDA path: ``csrc/optim.cu``; CPU path: the same arithmetic in PyTorch.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from ._lib import c_float, c_int, c_ll, check, ptr, stream


def sumsq_accumulate(g: torch.Tensor, out: torch.Tensor) -> None:
    """``out[0] += sum(g^2)`` (``out`` fp32, zeroed by the caller beforehand)."""
    if _lib.use_kernels(g, out) and g.dtype in (torch.bfloat16, torch.float32) and g.is_contiguous():
        # block partials are added in index order: the norm is the same bit pattern on every run
        from .elementwise import _workspace
        part = _workspace("sumsq_partials", 4096, g.device)
        check(_lib.load().msrl_sumsq_ordered(ptr(g), c_int(1 if g.dtype == torch.bfloat16 else 0),
                                             c_ll(g.numel()), ptr(part), c_int(4096), ptr(out), stream()), "sumsq")
        return
    out.add_(g.float().pow(2).sum())


def clip_coefficient(sumsq: torch.Tensor, max_norm: float, extra_scale: float, coef: torch.Tensor,
                     norm_out: torch.Tensor) -> None:
    """``coef = min(1, max_norm/(sqrt(sumsq)+1e-6)) * extra_scale`` without leaving the device."""
    if _lib.use_kernels(sumsq, coef, norm_out):
        check(_lib.load().msrl_clip_coef(ptr(sumsq), c_float(max_norm), c_float(extra_scale), ptr(coef),
                                         ptr(norm_out), stream()), "clip_coef")
        return
    norm = sumsq.sqrt()
    c = torch.clamp(max_norm / (norm + 1e-6), max=1.0) if max_norm > 0 else torch.ones_like(norm)
    coef.copy_((c * extra_scale).reshape(coef.shape))
    norm_out.copy_(norm.reshape(norm_out.shape))


def adamw_step(p32: torch.Tensor, m: torch.Tensor, v: torch.Tensor, g: torch.Tensor,
               p16: Optional[torch.Tensor], lr: float, beta1: float, beta2: float, eps: float,
               weight_decay: float, step: int, grad_scale: Optional[torch.Tensor] = None) -> None:
    """One decoupled-weight-decay Adam step on flat buffers.

    ``p32/m/v`` fp32 master state, ``g`` bf16 or fp32 gradient, ``p16`` optional bf16 working
    copy refreshed in the same pass, ``grad_scale`` optional 1-element device tensor (clip
    coefficient x 1/accumulation).
    """
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    if _lib.use_kernels(p32, m, v, g):
        check(_lib.load().msrl_adamw(ptr(p32), ptr(m), ptr(v), ptr(g),
                                     c_int(1 if g.dtype == torch.bfloat16 else 0), ptr(p16),
                                     c_ll(p32.numel()), c_float(lr), c_float(beta1), c_float(beta2),
                                     c_float(eps), c_float(weight_decay), c_float(bc1), c_float(bc2),
                                     ptr(grad_scale), stream()), "adamw")
        return
    gf = g.float()
    if grad_scale is not None:
        gf = gf * grad_scale.float()
    m.mul_(beta1).add_(gf, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(gf, gf, value=1 - beta2)
    p32.mul_(1 - lr * weight_decay).addcdiv_(m / bc1, (v / bc2).sqrt() + eps, value=-lr)
    if p16 is not None:
        p16.copy_(p32)


def cast_f32_to_bf16(src: torch.Tensor, dst: torch.Tensor) -> None:
    if _lib.use_kernels(src, dst):
        check(_lib.load().msrl_cast_f32_bf16(ptr(src), ptr(dst), c_ll(src.numel()), stream()), "cast")
        return
    dst.copy_(src)
