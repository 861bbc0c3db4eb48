"""Stand-alone model workers for disaggregated deployments and PPO: reference, critic, reward.

Each owns one model (no rollout engine) and runs the common stage loop against the experience
store.  Between its stages a worker can park its state in pinned host memory so that co-located
roles time-share the GPU (reference: ``workers/reference_worker.py:25-196``,
``workers/critic_worker.py:84-326``, ``workers/reward_worker.py:27-186``).
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional

import torch

from ..models.gpt import GPTModel
from ..models.training_engine import TrainingEngine
from ..models.transformer_config import TransformerConfig
from ..optim.optimizer_config import OptimizerConfig
from ..parallel.ddp import DistributedDataParallel, expert_replica_groups
from ..parallel.tp_comm import TPComm
from ..reshard.sharding_manager import GradBufferOffloader, ParamOffloader
from .base_worker import BaseWorker, profiled_stage


class _ModelWorker(BaseWorker):
    role = "reference"
    trainable = False
    value_head = False

    def __init__(self, megatron_config, rl_config, generate_config=None, td=None, *, pad_token_id: int = 0,
                 device=None, seed: Optional[int] = None, offload_between_stages: bool = False,
                 init_from: Optional[GPTModel] = None):
        super().__init__(td, pad_token_id)
        self.megatron_config, self.rl_config, self.generate_config = megatron_config, rl_config, generate_config
        self.device = torch.device(device if device is not None
                                   else ("cuda" if torch.cuda.is_available() else "cpu"))
        self.seed = megatron_config.seed if seed is None else seed
        self.offload_between_stages = offload_between_stages
        self.init_from = init_from
        self.iteration = 0
        self.consumed_train_samples = 0

    def initialize(self) -> None:
        mc, rl = self.megatron_config, self.rl_config
        ps = self.parallel_state
        tp = ps.size("tp")
        self.comm = TPComm(ps.group("tp"), mc.sequence_parallel, world_size=tp, rank=ps.rank_in("tp"))
        dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        tcfg = TransformerConfig.from_megatron(mc, params_dtype=dtype, value_head=self.value_head)
        self.tcfg = tcfg
        core = GPTModel(tcfg, self.comm, device=self.device, seed=self.seed)
        if self.init_from is not None:
            core.load_state_dict(self.init_from.state_dict(), strict=False)
        if mc.load and not self.trainable:
            from ..checkpoint.mcore import load_checkpoint

            load_checkpoint(mc.load, core, None, None, ps, mc, strict=not self.value_head)
        dp = ps.size("dp_cp")
        temperature = 1.0
        if self.generate_config is not None:
            temperature = self.generate_config.sampling_config.get("temperature", 1.0) or 1.0
        common = dict(stage=mc.stage or "ray_grpo", temperature=temperature, use_dynamic_bsz=rl.use_dynamic_bsz,
                      pad_multiple=tp * ps.size("cp"), dp_group=ps.group("dp_cp"), dp_size=dp,
                      device=self.device, micro_batch_size=mc.micro_batch_size or 1,
                      max_packing_token_size=rl.max_packing_token_size)
        if self.trainable:
            self.model = DistributedDataParallel(core, ps.group("dp_cp"), dp,
                                                 grad_in_fp32=bool(mc.accumulate_allreduce_grads_in_fp32),
                                                 **expert_replica_groups(ps, tcfg))
            self.model.attach_tensor_parallel(ps.group("tp"), tp, bool(mc.sequence_parallel))
            self.optimizer, self.scheduler = OptimizerConfig.from_training_config(mc).build(
                self.model.buffers, dp_group=ps.group("dp_cp"), dp_rank=ps.rank_in("dp_cp"),
                model_parallel_group=ps.group("mp"), tp_rank=ps.rank_in("tp"),
                total_steps=max(mc.train_iters or 1, 1), warmup_steps=0, default_lr=1e-6)
            if mc.load:
                # trainable roles (the critic) resume with their optimizer state, schedule and step count; a
                # checkpoint without a value head (fine-tuning from a policy) loads loosely and starts at step 0
                from ..checkpoint.mcore import load_checkpoint

                self.iteration, self.consumed_train_samples = load_checkpoint(
                    mc.load, core, self.optimizer, self.scheduler, ps, mc, strict=not self.value_head)
            self.engine = TrainingEngine(self.model, self.optimizer, self.scheduler, role=self.role,
                                         mini_batch_size_per_dp=max(rl.mini_batch_size // dp, 1),
                                         epochs=rl.epochs, shuffle_mini_batch=rl.shuffle_mini_batch,
                                         cliprange_value=rl.cliprange_value, **common)
            self.param_offloader = ParamOffloader(self.model)
            self.grad_offloader = GradBufferOffloader(self.model)
        else:
            for p in core.parameters():
                p.requires_grad_(False)
            self.model = core
            self.optimizer = self.scheduler = None
            self.engine = TrainingEngine(core, role=self.role, **common)
            self.param_offloader = self.grad_offloader = None
        if self.offload_between_stages:
            self._offload()

    # ---- memory -----------------------------------------------------------------------------------
    def _onload(self) -> None:
        if self.param_offloader is not None:
            self.param_offloader.onload()
            self.grad_offloader.restore()
            self.optimizer.onload_state()
        elif self.offload_between_stages and getattr(self, "_parked", False):
            self.model.to(self.device)
            self._parked = False

    def _offload(self) -> None:
        if not self.offload_between_stages:
            return
        if self.param_offloader is not None:
            self.grad_offloader.release()
            self.optimizer.offload_state()
            self.param_offloader.offload()
        else:
            self.model.to("cpu")
            self._parked = True

    def init_transfer_dock(self, td, mm_td=None, sampling_transfer_dock=None) -> None:
        self.td = td

    def get_iteration(self) -> int:
        return self.iteration

    def get_consumed_train_samples(self) -> int:
        return self.consumed_train_samples

    # ---- generic forward stage ------------------------------------------------------------------------
    def _forward_stage(self, consumer: str, out_column: str, dispatch_size: int, timing_key: str,
                       ragged: bool = True) -> None:
        columns = ["input_ids", "responses", "response_length", "prompt_length"]
        self._onload()
        start = time.time()
        while True:
            batch, idx, finished = self.dispatch_transfer_dock_data(
                consumer, columns, dispatch_size, get_n_samples=False,
                use_batch_seqlen_balance=self.rl_config.use_dp_batch_balance)
            if finished:
                break
            if batch is None:
                time.sleep(0.002)
                continue
            out = self.engine.forward(batch)
            self.collect_transfer_dock_data({out_column: out}, idx,
                                            lengths=batch["response_length"] if ragged else None)
        end = time.time()
        self.update_metrics(timing_key, [round(end, 4), round(start, 4)])
        self._offload()

    def save_checkpoint(self, iteration: int) -> None:
        from ..checkpoint.mcore import save_checkpoint

        if not self.megatron_config.save or not self.trainable:
            return
        self._onload()
        save_checkpoint(self.megatron_config.save, iteration, self.model.module, self.optimizer, self.scheduler,
                        self.parallel_state, self.megatron_config,
                        consumed_train_samples=self.consumed_train_samples)
        self._offload()


class ReferenceWorker(_ModelWorker):
    """Frozen policy copy -> ``ref_log_prob``."""
    role = "reference"

    @profiled_stage("reference_compute_log_prob")
    def compute_ref_log_prob(self) -> None:
        self._forward_stage("ref_log_prob", "ref_log_prob", self.rl_config.ref_dispatch_size,
                            "timing/reference_model")
        self.update_metrics("end_time/reference", [round(time.time(), 4)])


class RewardWorker(_ModelWorker):
    """Outcome reward model: value-head output at the last token -> ``rm_scores``."""
    role = "reward"
    value_head = True

    def compute_rm_score(self) -> None:
        self._forward_stage("reward_scores", "rm_scores", self.rl_config.reward_dispatch_size,
                            "timing/reward_model", ragged=False)


class CriticWorker(_ModelWorker):
    """Value model: ``compute_values`` and the clipped value-loss update."""
    role = "critic"
    trainable = True
    value_head = True

    @profiled_stage("critic_compute_values")
    def compute_values(self) -> None:
        self._forward_stage("critic_compute_values", "values", self.rl_config.critic_value_dispatch_size,
                            "timing/critic_model")

    @profiled_stage("critic_update")
    def update_critic(self) -> None:
        rl = self.rl_config
        columns = ["responses", "advantages", "values", "returns", "input_ids", "response_length", "prompt_length"]
        self._onload()
        start = time.time()
        while True:
            batch, idx, finished = self.dispatch_transfer_dock_data(
                "critic_train", columns, rl.critic_update_dispatch_size, get_n_samples=False,
                use_batch_seqlen_balance=rl.use_dp_batch_balance)
            if finished:
                break
            if batch is None:
                time.sleep(0.002)
                continue
            metrics = self.engine.update(batch)
            self.dump_key_data("critic_update", "critic_train_dump",
                               {**{k: batch[k] for k in ("values", "returns", "advantages") if k in batch},
                                **{k: (sum(v) / len(v) if isinstance(v, (list, tuple)) and v else v)
                                   for k, v in metrics.items() if k.startswith("critic/")}})
            self.consumed_train_samples += len(idx) * self.parallel_state.size("dp_cp")
            if self.is_writer():
                self.td.update_metrics("", value=metrics, cumulate=True)
        self.update_metrics("timing/update_critic", [round(time.time(), 4), round(start, 4)])
        self.iteration += 1
        self._offload()

    update = update_critic
