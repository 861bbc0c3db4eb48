"""Shared driver-loop machinery of the RL trainers (GRPO / DAPO / PPO).

Holds the worker groups, the KL controller, the experience store handle, logging sinks and the
checkpoint trigger (reference: ``mindspeed_rl/trainer/base.py:14-112``).  The experience store
lives in the driver process (rank 0) and is served to the other ranks through ``runtime.rpc``.
"""
from __future__ import annotations

import os
import time
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

from ..data.transfer_dock import GRPOTransferDock
from ..obs.loggers import Loggers, SwanLabLogger, WandbLogger
from ..obs.metrics import Metric
from ..runtime import rpc
from .compute_utils import get_kl_controller


class RayBaseTrainer:
    def __init__(self, actor_worker=None, ref_worker=None, reward_list: Optional[List[Any]] = None,
                 critic_worker=None, train_iters: int = 1, save_interval: int = 1,
                 gamma: float = 1.0, lam: float = 0.95, adv_estimator: str = "group_norm",
                 missing_eos_penalty: float = 1.0, kl_penalty: str = "low_var_kl",
                 kl_ctrl_type: str = "fixed", kl_horizon: int = 1000, kl_target: float = 100.0,
                 init_kl_coef: float = 0.01, global_batch_size: int = 1, micro_batch_size: int = 1,
                 n_samples_per_prompt: int = 1, tokenizer=None, dataset_additional_keys=None,
                 blocking: bool = True, guarantee_order: bool = False, num_cpus_for_local_task: int = 1,
                 partial_rollout_max_split: int = 1, use_kl_in_reward: bool = False,
                 use_tensorboard: bool = False, use_wandb: bool = False, use_swanlab: bool = False,
                 pad_token_id: Optional[int] = None, **kwargs):
        self.actor_worker, self.ref_worker = actor_worker, ref_worker
        self.critic_worker = critic_worker
        self.reward_list = reward_list or []
        self.train_iters, self.save_interval = train_iters, save_interval
        self.gamma, self.lam, self.adv_estimator = gamma, lam, adv_estimator
        self.missing_eos_penalty = missing_eos_penalty
        self.kl_penalty, self.kl_ctrl_type = kl_penalty, kl_ctrl_type
        self.kl_horizon, self.kl_target, self.init_kl_coef = kl_horizon, kl_target, init_kl_coef
        self.global_batch_size, self.micro_batch_size = global_batch_size, micro_batch_size
        self.n_samples_per_prompt = n_samples_per_prompt
        self.tokenizer = tokenizer
        self.dataset_additional_keys = list(dataset_additional_keys or [])
        self.blocking, self.guarantee_order = blocking, guarantee_order
        self.num_cpus_for_local_task = num_cpus_for_local_task
        self.partial_rollout_max_split = partial_rollout_max_split
        self.use_kl_in_reward = use_kl_in_reward
        self.kwargs = kwargs
        if pad_token_id is None and tokenizer is not None:
            pad = getattr(tokenizer, "pad", None)
            pad_token_id = pad if pad is not None else getattr(tokenizer, "eod", 0)
        self.pad_token_id = pad_token_id or 0
        self.kl_ctrl = get_kl_controller(kl_ctrl_type, init_kl_coef, kl_target, kl_horizon)
        self.logger = Loggers(name=type(self).__name__)
        self.tensorboard = None
        self.wandb = None
        self.swanlab = None
        self.is_driver = getattr(actor_worker, "is_driver", True)
        if self.is_driver:
            if use_wandb:
                self.wandb = WandbLogger(kwargs)
            elif use_tensorboard:
                try:
                    from torch.utils.tensorboard import SummaryWriter

                    self.tensorboard = SummaryWriter(kwargs.get("tensorboard_dir") or None)
                except Exception as e:  # pragma: no cover - optional sink
                    self.logger.warning(f"tensorboard unavailable: {e}")
            if use_swanlab:
                self.swanlab = SwanLabLogger(kwargs)
        self._td_server = None

    # ---- experience store plumbing ----------------------------------------------------------------
    def _new_dock(self, *args, **kwargs):
        """Driver side: build the experience store the run's ``data_strategy`` names
        (``td``: one in-process dock, ``tq``: metadata manager + tensor shards)."""
        from ..data.transfer_queue import DataStrategy

        rl = getattr(self.actor_worker, "rl_config", None)
        strategy = DataStrategy(getattr(rl, "data_strategy", "td") or "td",
                                getattr(rl, "transfer_queue_data_shard_num", 1) or 1)
        self._strategies = getattr(self, "_strategies", []) + [strategy]
        dock, self._dock_descriptor = strategy.create(*args, **kwargs)
        return dock

    def _share_dock(self, dock, name: str = "td"):
        """Make the driver's dock reachable from every rank; returns this rank's handle."""
        from ..data.transfer_queue import DataStrategy

        world = dist.get_world_size() if (dist.is_available() and dist.is_initialized()) else 1
        descriptor = getattr(self, "_dock_descriptor", None) if self.is_driver else None
        self._dock_descriptor = None
        if world == 1:
            return DataStrategy.attach(dock, descriptor)
        box = [None, None]
        if self.is_driver:
            server = rpc.serve(dock, "tcp://127.0.0.1:0", num_threads=max(8, world * 2))
            self._servers = getattr(self, "_servers", []) + [server]
            box = [server.address, descriptor]
        dist.broadcast_object_list(box, src=0)
        return DataStrategy.attach(dock if self.is_driver else rpc.connect(box[0]), box[1])

    def _driver_section_done(self) -> None:
        """Host barrier after a driver-only stage."""
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            dist.barrier()

    # ---- logging -----------------------------------------------------------------------------------
    def log_metrics(self, metrics: Dict[str, Any], iteration: int, steps: int) -> None:
        if not self.is_driver:
            return
        self.logger.info(metrics, iteration, steps)
        if self.tensorboard is not None:
            for k, v in metrics.items():
                if isinstance(v, (int, float)):
                    self.tensorboard.add_scalar(k, v, iteration)
        if self.wandb is not None:
            self.wandb.log_metrics(metrics, iteration)
        if self.swanlab is not None:
            self.swanlab.log_metrics(metrics, iteration)

    def save_checkpoint(self, iteration: int) -> None:
        self.actor_worker.save_checkpoint(iteration)
        if self.critic_worker is not None:
            self.critic_worker.save_checkpoint(iteration)
