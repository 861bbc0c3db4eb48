"""GRPO driver loop.

One iteration (reference: ``mindspeed_rl/trainer/grpo_trainer_hybrid.py:175-295``):
prompts -> store (n copies each) -> rollout -> rule / model reward -> group-normalised
advantages -> reference log-probs -> (old log-probs unless one on-policy update) -> policy
update -> metrics (timings, throughput, scores) -> clear the store -> checkpoint.
"""
from __future__ import annotations

import time
from typing import Any, Dict, Iterator, List, Optional

import torch

from ..data.transfer_dock import GRPOTransferDock, put_prompts_experience
from ..obs.metrics import Metric, compute_tps, metrics_post_processing, metrics_sort
from ..utils.pad_process import padding_dict_to_tensor_dict
from .base import RayBaseTrainer
from .compute_utils import compute_advantage, compute_grpo_data_metrics


class RayGRPOTrainer(RayBaseTrainer):
    def __init__(self, actor_worker, ref_worker=None, reward_list=None, vit_worker=None, **kw):
        super().__init__(actor_worker, ref_worker or actor_worker, reward_list, **kw)
        self.vit_worker = vit_worker          # vision-encoder stage of vision-language runs (or None)
        self.enable_partial_rollout = self.partial_rollout_max_split > 1
        self.metrics = Metric()
        self.td_max_len = self.global_batch_size * (2 if self.enable_partial_rollout else 1)
        self.transfer_dock = None
        self.transfer_dock_init()
        self.set_actor_log_prob_skip_flag()

    # ------------------------------------------------------------------------------------------
    def transfer_dock_init(self) -> None:
        dock = None
        cols = list(self.dataset_additional_keys)
        if getattr(getattr(self.actor_worker, "rl_config", None), "multi_turn_enable", False):
            cols += ["response_mask", "tool_call_num"]          # written by the multi-turn rollout loop
        if self.is_driver:
            dock = self._new_dock(self.td_max_len, self.n_samples_per_prompt, self.metrics,
                                  max_age=self.partial_rollout_max_split, GBS_train=self.global_batch_size,
                                  addition_columns=cols)
        self.transfer_dock = self._share_dock(dock)
        self.mm_transfer_dock = None
        rl = getattr(self.actor_worker, "rl_config", None)
        if rl is not None and rl.is_multimodal:
            from ..data.mm_transfer_dock import MMGRPOTransferDock

            mm = MMGRPOTransferDock(self.td_max_len, self.n_samples_per_prompt, rl.reuse_image_embeds) \
                if self.is_driver else None
            self._dock_descriptor = None
            self.mm_transfer_dock = self._share_dock(mm, "mm_td")
        self.actor_worker.sync_init_transfer_dock(self.transfer_dock, self.mm_transfer_dock)
        if self.vit_worker is not None:
            self.vit_worker.sync_init_transfer_dock(self.transfer_dock, self.mm_transfer_dock)
        if self.ref_worker is not self.actor_worker:
            self.ref_worker.sync_init_transfer_dock(self.transfer_dock, self.mm_transfer_dock)
        for r in self.reward_list:
            (getattr(r, "sync_init_transfer_dock", None) or r.init_transfer_dock)(self.transfer_dock)

    def set_actor_log_prob_skip_flag(self) -> None:
        rl = self.actor_worker.rl_config
        gbs = self.actor_worker.megatron_config.global_batch_size
        self.skip_actor_log_prob = (gbs * rl.n_samples_per_prompt == rl.mini_batch_size and rl.epochs == 1)

    # ------------------------------------------------------------------------------------------
    def fit(self, data_iters: Iterator[Dict[str, List[torch.Tensor]]]) -> List[Dict[str, Any]]:
        """Run ``train_iters`` iterations; returns the logged metrics of every iteration."""
        rl = self.actor_worker.rl_config
        td = self.transfer_dock
        iteration = self.actor_worker.get_iteration()
        history = []
        if self.enable_partial_rollout and self.is_driver:
            first = next(data_iters)
            data, idx = put_prompts_experience(first, self.n_samples_per_prompt, self.dataset_additional_keys)
            td.put_experience(padding_dict_to_tensor_dict(data), idx, is_prompt=True)
        while iteration < self.train_iters:
            t0 = time.time()
            if self.is_driver:
                batch = next(data_iters)
                data, idx = put_prompts_experience(batch, self.n_samples_per_prompt,
                                                   self.dataset_additional_keys,
                                                   add_another_batch=self.enable_partial_rollout)
                td.put_experience(padding_dict_to_tensor_dict(data), idx, is_prompt=True)
                if self.mm_transfer_dock is not None and batch.get("mm"):
                    n_prompts = len(batch["prompts"])
                    first = idx[0] // self.n_samples_per_prompt
                    self.mm_transfer_dock.put_experience(batch["mm"], list(range(first, first + n_prompts)))
            self._driver_section_done()
            # vision-language runs: the vision tower runs once per prompt, everyone else reads its output
            if self.vit_worker is not None:
                self.vit_worker.compute_image_embeds(blocking=True)
                self._driver_section_done()
            # rollout
            self.actor_worker.generate_sequences(blocking=self.blocking)
            if self.enable_partial_rollout:
                # the set of completed groups must stand still before any stage picks its rows: a replica that
                # is still writing results would shift the window the other stages have already started on
                self.actor_worker.barrier()
            # model-based reward scorers are stages of a worker group: every rank of the job makes the call
            for reward in self.reward_list:
                if hasattr(reward, "worker"):
                    reward.compute_rm_score(blocking=True)
            # rule rewards + advantages (driver-side CPU stages)
            if self.is_driver:
                t_r = time.time()
                for reward in self.reward_list:
                    if not hasattr(reward, "worker"):
                        reward.compute_rm_score()
                t_a = time.time()
                compute_advantage(td, self.gamma, self.lam, self.adv_estimator, rl.adv_dispatch_size,
                                  self.pad_token_id, self.global_batch_size, self.guarantee_order,
                                  self.n_samples_per_prompt, multi_turn_enable=rl.multi_turn_enable)
                t_e = time.time()
                td.update_metrics("timing/adv", value=[round(t_e, 4), round(t_a, 4)], cumulate=True)
                td.update_metrics("end_time/end_adv_time", value=[round(t_e, 4)], cumulate=True)
            self._driver_section_done()
            # reference + old log-probs
            if self.ref_worker is not None and getattr(self.ref_worker.worker, "with_reference", True):
                td.update_metrics("start_time/reference_model", value=[round(time.time(), 4)], cumulate=True) \
                    if self.is_driver else None
                self.ref_worker.compute_ref_log_prob(blocking=self.blocking)
            if not self.skip_actor_log_prob:
                self.actor_worker.compute_log_prob(blocking=self.blocking)
            self.actor_worker.wait_all_ref_objs_run_over()
            # update
            self.actor_worker.update(self.kl_ctrl, self.skip_actor_log_prob)
            self._driver_section_done()
            iteration += 1
            if self.is_driver:
                data_metrics = compute_grpo_data_metrics(td, self.global_batch_size * self.n_samples_per_prompt,
                                                         self.pad_token_id, self.global_batch_size,
                                                         self.guarantee_order,
                                                         multi_turn_enable=rl.multi_turn_enable)
                m = metrics_post_processing(td.get_metrics())
                m.update(data_metrics)
                time_all = time.time() - t0
                m = metrics_sort(m, time_all)
                kw = dict(actor_resource=rl.actor_resource, reference_resource=rl.reference_resource,
                          reward_resource=rl.reward_resource, use_integrated_worker=rl.use_integrated_worker)
                gbs, n = self.global_batch_size, self.n_samples_per_prompt
                m["e2e_tps"] = compute_tps(kw, m, gbs, n, time_all, rl.log_max_throughput)
                if m.get("timing/update"):
                    m["update_tps"] = compute_tps(kw, m, gbs, n, m["timing/update"], rl.log_max_throughput)
                if m.get("timing/rollout"):
                    m["vllm_tps"] = compute_tps(kw, m, gbs, n, m["timing/rollout"], rl.log_max_throughput)
                self.log_metrics(m, iteration, self.train_iters)
                history.append(m)
                td.clear()
                if self.mm_transfer_dock is not None:
                    self.mm_transfer_dock.clear()
            self._driver_section_done()
            if self.save_interval and (iteration % self.save_interval == 0 or iteration == self.train_iters):
                self.save_checkpoint(iteration)
        return history
