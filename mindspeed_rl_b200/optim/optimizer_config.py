"""``OptimizerConfig``: the optimizer knobs of a training config as one typed object.

Mirrors the attribute names Megatron's optimizer config uses (reference:
``mindspeed_rl/utils/optimizer_module.py:10-119``), so recipes written for the reference carry over;
``from_training_config`` picks them off an actor / critic config and ``build`` turns them into
this repository's ZeRO-1 ``DistributedOptimizer`` plus its learning-rate schedule.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Any, Optional

import torch


@dataclass
class OptimizerConfig:
    optimizer: str = "adam"
    lr: Optional[float] = None
    min_lr: Optional[float] = None
    decoupled_lr: Optional[float] = None
    decoupled_min_lr: Optional[float] = None
    weight_decay: float = 0.01
    fp16: bool = False
    bf16: bool = False
    params_dtype: torch.dtype = torch.float32
    loss_scale: Optional[float] = None
    initial_loss_scale: float = 2.0 ** 32
    min_loss_scale: float = 1.0
    loss_scale_window: float = 1000.0
    hysteresis: int = 2
    adam_beta1: float = 0.9
    adam_beta2: float = 0.999
    adam_eps: float = 1e-08
    sgd_momentum: float = 0.9
    use_distributed_optimizer: bool = False
    overlap_grad_reduce: bool = False
    overlap_param_gather: bool = False
    clip_grad: float = 1.0
    log_num_zeros_in_grad: bool = False
    barrier_with_L1_time: bool = False
    # host-offloaded state and the 16-bit-residual master weights (MindSpeed features)
    swap_optimizer: bool = False
    swap_optimizer_times: int = 16
    reuse_fp32_param: bool = False
    # schedule
    lr_decay_style: str = "constant"
    lr_warmup_fraction: Optional[float] = None
    lr_warmup_iters: int = 0
    lr_decay_iters: Optional[int] = None
    train_iters: Optional[int] = None

    @classmethod
    def from_training_config(cls, cfg: Any) -> "OptimizerConfig":
        """Every field that ``cfg`` (attribute bag or dict) defines; the rest keep their defaults."""
        get = (lambda k: cfg.get(k)) if isinstance(cfg, dict) else (lambda k: getattr(cfg, k, None))
        kw = {}
        for f in dataclasses.fields(cls):
            v = get(f.name)
            if v is not None:
                kw[f.name] = v
        out = cls(**kw)
        if out.bf16:
            out.params_dtype = torch.bfloat16
        if out.optimizer not in ("adam", "fused_adamw", "adamw"):
            raise ValueError(f"optimizer {out.optimizer!r} is not supported (adam / adamw / fused_adamw)")
        return out

    def build(self, buffers, dp_group=None, dp_rank: int = 0, model_parallel_group=None, tp_rank: int = 0,
              total_steps: Optional[int] = None, warmup_steps: Optional[int] = None, default_lr: float = 0.0):
        """``(DistributedOptimizer, OptimizerParamScheduler)`` for the flat parameter buffers of a model.
        ``total_steps`` / ``warmup_steps`` give the schedule's length in the unit the caller steps it
        with (the RL workers count samples); by default they come from the iteration fields."""
        from .distributed_optimizer import DistributedOptimizer, OptimizerParamScheduler

        lr = self.lr if self.lr else default_lr
        opt = DistributedOptimizer(
            buffers, lr=lr, betas=(self.adam_beta1, self.adam_beta2), eps=self.adam_eps,
            weight_decay=self.weight_decay, clip_grad=self.clip_grad, dp_group=dp_group, dp_rank=dp_rank,
            model_parallel_group=model_parallel_group, offload_to_host=self.swap_optimizer,
            swap_chunks=self.swap_optimizer_times, tp_rank=tp_rank, reuse_fp32_param=self.reuse_fp32_param,
            overlap_param_gather=self.overlap_param_gather)
        total = total_steps if total_steps is not None else (self.lr_decay_iters or self.train_iters or 0)
        if warmup_steps is not None:
            warm = warmup_steps
        else:
            warm = self.lr_warmup_iters or int((self.lr_warmup_fraction or 0.0) * total)
        sched = OptimizerParamScheduler(opt, lr, self.min_lr or 0.0, warm, total, self.lr_decay_style or "constant")
        return opt, sched
