"""Loss registry keyed by ``"{stage}_{role}"`` and the loss classes of every stage / role.

Stages ``ray_grpo | ray_dapo | ray_ppo``, roles ``actor | reference | reward | critic``
(reference: ``mindspeed_rl/models/loss/loss_register.py:4-23`` and the ``*_loss_func.py`` files
next to it).  A loss object receives the per-token response tensors and returns the gradient
with respect to the model output of its role -- every objective is evaluated forward *and*
backward by one fused kernel (``ops.policy_loss_fwd_bwd`` / ``ops.value_loss_fwd_bwd``), so no
autograd graph is built over the ``[B, L]`` tensors.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional, Tuple

import torch

from ... import ops
from ...utils.torch_functional import sequence_mask


class LossRegister:
    class_map: Dict[str, type] = {}

    @classmethod
    def register_loss(cls, stage: str, role: str) -> Callable[[type], type]:
        def deco(klass: type) -> type:
            cls.class_map[f"{stage}_{role}"] = klass
            return klass
        return deco

    @classmethod
    def get_instance(cls, stage: str, role: str, **kw):
        key = f"{stage}_{role}"
        if key not in cls.class_map:
            raise ValueError(f"no loss registered for stage '{stage}' and role '{role}'")
        return cls.class_map[key](**kw)


class LossFuncFactory(LossRegister):
    class_map: Dict[str, type] = {}


class BaseLossFunc:
    """Common helpers: response mask and metric bookkeeping."""

    needs_backward = True
    output_kind = "logprob"   # "logprob" -> (logp, entropy) per response token; "value" -> scalars

    def __init__(self, **kw):
        self.options = dict(kw)

    def add_loss_meta_info(self, meta_info: Optional[dict]) -> None:
        if meta_info:
            self.options.update(meta_info)

    @staticmethod
    def response_mask(batch: dict, width: int, device) -> torch.Tensor:
        if batch.get("response_mask") is not None:
            return batch["response_mask"].to(device).float()
        return sequence_mask(batch["response_length"].to(device), width)


def _opt(batch, key, device):
    v = batch.get(key)
    return None if v is None else v.to(device).float()


class _ActorLoss(BaseLossFunc):
    """Shared machinery of the three actor objectives."""

    use_kl = False

    def clip_range(self) -> Tuple[float, float]:
        c = self.options.get("clip_ratio", 0.2)
        return c, c

    def token_level(self) -> bool:
        return True

    def compute(self, batch: dict, logp: torch.Tensor, entropy: Optional[torch.Tensor],
                loss_scale: float = 1.0):
        """Returns ``(dlogp, dentropy_or_None, stats)``; all ``[B, L]`` / 0-dim device tensors."""
        dev = logp.device
        mask = self.response_mask(batch, logp.shape[1], dev)
        lo, hi = self.clip_range()
        kl_coef = float(self.options.get("kl_ctrl", 0.0) or 0.0) if self.use_kl else 0.0
        ref = _opt(batch, "ref_log_prob", dev) if self.use_kl else None
        dlogp, st = ops.policy_loss_fwd_bwd(
            logp, _opt(batch, "old_log_prob", dev), ref, batch["advantages"].to(dev).float(), mask, lo, hi,
            kl_coef, self.options.get("kl_penalty", "low_var_kl") if self.use_kl else None,
            self.token_level(), loss_scale)
        stats = {"actor/pg_loss": st["pg_loss"], "actor/pg_clipfrac": st["pg_clipfrac"],
                 "actor/ppo_kl": st["ppo_kl"], "actor/kl_loss": st["kl_loss"]}
        dent = None
        c_ent = float(self.options.get("entropy_coeff", 0.0) or 0.0)
        if entropy is not None:
            w = ops.loss_weights(mask, True)
            stats["actor/entropy"] = (entropy.detach() * w).sum()
            if c_ent != 0.0:
                dent = -c_ent * loss_scale * w
        return dlogp, dent, stats


@LossFuncFactory.register_loss("ray_grpo", "actor")
class GRPOActorLossFunc(_ActorLoss):
    """Clipped surrogate + ``kl_ctrl * KL(pi || ref)`` - ``entropy_coeff * H``."""
    use_kl = True


@LossFuncFactory.register_loss("ray_ppo", "actor")
class PPOActorLossFunc(_ActorLoss):
    """Clipped surrogate without KL term (KL enters through the reward)."""


@LossFuncFactory.register_loss("ray_dapo", "actor")
class DAPOActorLossFunc(_ActorLoss):
    """Decoupled clip range (clip-higher), token-level or sequence-mean aggregation, no KL."""

    def clip_range(self):
        o = self.options
        if o.get("clip_higher_enable", False):
            return o.get("clip_ratio_low", 0.2), o.get("clip_ratio_high", 0.28)
        c = o.get("clip_ratio", 0.2)
        return c, c

    def token_level(self):
        return bool(self.options.get("token_level_loss", True))


class _ForwardOnly(BaseLossFunc):
    needs_backward = False

    def compute(self, batch, logp, entropy, loss_scale: float = 1.0):
        return None, None, {}


for _stage in ("ray_grpo", "ray_ppo", "ray_dapo"):
    LossFuncFactory.register_loss(_stage, "reference")(type("ReferenceLossFunc", (_ForwardOnly,), {
        "__doc__": "Reference model: log-probabilities only."}))
    LossFuncFactory.register_loss(_stage, "reward")(type("RewardLossFunc", (_ForwardOnly,), {
        "__doc__": "Reward model: scores only.", "output_kind": "value"}))


@LossFuncFactory.register_loss("ray_ppo", "critic")
class CriticLossFunc(BaseLossFunc):
    """``0.5 * mean(max((v - R)^2, (clip(v, v_old +- c) - R)^2))``."""
    output_kind = "value"

    def compute(self, batch, vpreds: torch.Tensor, _unused=None, loss_scale: float = 1.0):
        dev = vpreds.device
        mask = self.response_mask(batch, vpreds.shape[1], dev)
        dv, st = ops.value_loss_fwd_bwd(vpreds, batch["values"].to(dev).float(),
                                        batch["returns"].to(dev).float(), mask,
                                        float(self.options.get("cliprange_value", 0.5)), loss_scale)
        return dv, None, {"critic/vf_loss": st["vf_loss"].abs(), "critic/vf_clipfrac": st["vf_clipfrac"]}
