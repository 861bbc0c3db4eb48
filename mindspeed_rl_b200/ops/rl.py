"""RL objective ops: fused policy loss (forward + gradient in one pass), clipped value loss,
GAE and group-normalised advantages.

CUDA path: ``csrc/rl_math.cu``.  The PyTorch formulations below are the numerics oracle and
the CPU path; they spell out the reference formulas
(``mindspeed_rl/models/loss/grpo_actor_loss_func.py:100-144``,
``dapo_actor_loss_func.py:105-152``, ``ppo_actor_loss_func.py:91-132``,
``critic_loss_func.py:82-111``, ``trainer/utils/compute_utils.py:107-191``).
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from . import guard

from . import _lib
from ._lib import c_float, c_int, c_ll, check, ptr, stream
from ..utils.compute import compute_kl_penalty
from ..utils.torch_functional import masked_mean, masked_whiten

KL_KINDS = {None: 0, "none": 0, "kl": 1, "abs": 2, "mse": 3, "low_var_kl": 4}


def loss_weights(mask: torch.Tensor, token_level: bool = True) -> torch.Tensor:
    """Per-token weights that turn a sum into the masked mean used by the losses.

    token-mean: ``mask / (sum(mask) + 1e-8)``; seq-mean-token-mean: ``mask / sum_row(mask) / B``.
    """
    m = mask.float()
    if token_level:
        return m / (m.sum() + 1e-8)
    return m / m.sum(dim=-1, keepdim=True).clamp(min=1e-8) / m.shape[0]


def policy_loss_reference(logp, old_logp, ref_logp, adv, mask, clip_low, clip_high, kl_coef,
                          kl_penalty, token_level=True):
    """Differentiable PyTorch formulation (oracle). Returns (loss, stats dict)."""
    old = logp.detach() if old_logp is None else old_logp
    neg_kl = logp - old
    ratio = torch.exp(neg_kl)
    l1 = -adv * ratio
    l2 = -adv * torch.clamp(ratio, 1.0 - clip_low, 1.0 + clip_high)
    per_tok = torch.max(l1, l2)
    if token_level:
        pg = masked_mean(per_tok, mask)
    else:
        pg = ((per_tok * mask).sum(-1) / mask.sum(-1)).mean()
    stats = {
        "pg_loss": pg.detach(),
        "pg_clipfrac": masked_mean(torch.gt(l2, l1).float(), mask).detach(),
        "ppo_kl": masked_mean(-neg_kl, mask).detach(),
    }
    loss = pg
    if ref_logp is not None and kl_penalty not in (None, "none"):
        kl = masked_mean(compute_kl_penalty(logp, ref_logp, kl_penalty), mask)
        stats["kl_loss"] = kl.detach()
        loss = loss + kl_coef * kl
    else:
        stats["kl_loss"] = torch.zeros_like(pg.detach())
    return loss, stats


def policy_loss_fwd_bwd(logp: torch.Tensor, old_logp: Optional[torch.Tensor],
                        ref_logp: Optional[torch.Tensor], adv: torch.Tensor, mask: torch.Tensor,
                        clip_low: float, clip_high: float, kl_coef: float = 0.0,
                        kl_penalty: Optional[str] = None, token_level: bool = True,
                        loss_scale: float = 1.0) -> Tuple[torch.Tensor, Dict[str, torch.Tensor]]:
    """Evaluate the clipped objective and ``d loss / d logp`` in one pass.

    Returns ``(dlogp, stats)`` with ``stats = {loss, pg_loss, pg_clipfrac, ppo_kl, kl_loss}`` as
    0-dim tensors on the device of the inputs (no host sync).  ``loss_scale`` multiplies both the
    loss and the gradient (dynamic-batch re-weighting, gradient-accumulation scaling).
    """
    use_kl = ref_logp is not None and kl_penalty not in (None, "none")
    if _lib.use_kernels(logp, adv, mask):
        lp = logp.detach().float().contiguous()
        w_loss = (loss_weights(mask, token_level) * loss_scale).contiguous()
        w_stat = loss_weights(mask, True).contiguous()
        dlogp = guard.empty_like(lp)
        st = guard.empty(4, device=lp.device, dtype=torch.float32)
        old = old_logp.float().contiguous() if old_logp is not None else None
        ref = ref_logp.float().contiguous() if use_kl else None
        check(_lib.load().msrl_policy_loss(ptr(lp), ptr(old), ptr(ref), ptr(adv.float().contiguous()),
                                           ptr(w_loss), ptr(w_stat), ptr(dlogp), ptr(st),
                                           c_ll(lp.numel()), c_float(1.0 - clip_low),
                                           c_float(1.0 + clip_high), c_float(kl_coef if use_kl else 0.0),
                                           c_float(loss_scale),
                                           c_int(KL_KINDS[kl_penalty] if use_kl else 0), stream()),
              "policy_loss")
        pg = st[0] / loss_scale if loss_scale != 1.0 else st[0]
        stats = {"pg_loss": pg, "pg_clipfrac": st[1], "ppo_kl": st[2], "kl_loss": st[3],
                 "loss": st[0] + kl_coef * loss_scale * st[3]}
        return dlogp, stats
    with torch.enable_grad():
        x = logp.detach().float().requires_grad_(True)
        loss, stats = policy_loss_reference(x, old_logp, ref_logp if use_kl else None, adv.float(),
                                            mask.float(), clip_low, clip_high, kl_coef,
                                            kl_penalty if use_kl else None, token_level)
        loss = loss * loss_scale
        (dlogp,) = torch.autograd.grad(loss, x)
    stats["loss"] = loss.detach()
    return dlogp, stats


def value_loss_reference(vpreds, values, returns, mask, clip):
    vclip = torch.clamp(vpreds, values - clip, values + clip)
    l1 = (vpreds - returns) ** 2
    l2 = (vclip - returns) ** 2
    loss = 0.5 * masked_mean(torch.max(l1, l2), mask)
    frac = masked_mean(torch.gt(l2, l1).float(), mask)
    return loss, frac


def value_loss_fwd_bwd(vpreds, values, returns, mask, clip: float, loss_scale: float = 1.0):
    """Returns ``(dv, {"vf_loss", "vf_clipfrac"})``."""
    if _lib.use_kernels(vpreds, values, returns, mask):
        v = vpreds.detach().float().contiguous()
        w = (loss_weights(mask, True) * loss_scale).contiguous()
        dv = guard.empty_like(v)
        st = guard.empty(2, device=v.device, dtype=torch.float32)
        check(_lib.load().msrl_value_loss(ptr(v), ptr(values.float().contiguous()),
                                          ptr(returns.float().contiguous()), ptr(w), ptr(dv), ptr(st),
                                          c_ll(v.numel()), c_float(clip), stream()), "value_loss")
        return dv, {"vf_loss": st[0] / loss_scale, "vf_clipfrac": st[1] / loss_scale}
    with torch.enable_grad():
        x = vpreds.detach().float().requires_grad_(True)
        loss, frac = value_loss_reference(x, values.float(), returns.float(), mask.float(), clip)
        (dv,) = torch.autograd.grad(loss * loss_scale, x)
    return dv, {"vf_loss": loss.detach(), "vf_clipfrac": frac.detach()}


def gae(token_level_rewards: torch.Tensor, values: torch.Tensor, mask: torch.Tensor, gamma: float,
        lam: float, whiten: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """Generalised advantage estimation over ``[B, L]``; returns ``(advantages, returns)``.

    The reverse scan runs over the padded width without looking at the mask; the advantages are
    whitened over the masked tokens afterwards (reference: ``compute_utils.py:135-149``).
    """
    b, l = token_level_rewards.shape
    r, v = token_level_rewards.float().contiguous(), values.float().contiguous()
    if _lib.use_kernels(r, v):
        adv = guard.empty_like(r)
        ret = guard.empty_like(r)
        check(_lib.load().msrl_gae(ptr(r), ptr(v), ptr(adv), ptr(ret), c_int(b), c_int(l),
                                   c_float(gamma), c_float(lam), stream()), "gae")
    else:
        adv = torch.zeros_like(r)
        last = torch.zeros(b)
        nxt = torch.zeros(b)
        for t in range(l - 1, -1, -1):
            delta = r[:, t] + gamma * nxt - v[:, t]
            last = delta + gamma * lam * last
            adv[:, t] = last
            nxt = v[:, t]
        ret = adv + v
    if whiten:
        adv = masked_whiten(adv, mask.float())
    return adv, ret


def group_norm_advantage(scores: torch.Tensor, mask: torch.Tensor, n_samples: int,
                         eps: float = 1e-6) -> torch.Tensor:
    """``(s - mean_g) / (std_g + eps)`` per prompt group, broadcast over tokens and masked."""
    rows, l = mask.shape
    s = scores.reshape(-1).float().contiguous()
    if _lib.use_kernels(s, mask):
        adv = guard.empty(rows, l, device=mask.device, dtype=torch.float32)
        check(_lib.load().msrl_group_norm_adv(ptr(s), ptr(mask.float().contiguous()), ptr(adv),
                                              c_int(rows), c_int(n_samples), c_int(l), c_float(eps),
                                              stream()), "group_norm_adv")
        return adv
    g = s.double().reshape(-1, n_samples)
    a = ((g - g.mean(dim=1, keepdim=True)) / (g.std(dim=1, keepdim=True) + eps)).reshape(-1, 1)
    return (a.float() * mask.float())
