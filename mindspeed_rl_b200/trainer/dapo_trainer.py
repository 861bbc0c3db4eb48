"""DAPO driver loop: GRPO without reference model, clip-higher, token-level loss, overlong
shaping (in the rule reward) and *dynamic sampling*.

With ``filter_groups_enable`` two docks are used: rollouts and rewards land in the *sampling*
dock (one generation batch); ``DynamicSampling`` moves prompt groups whose reward is not
constant into the *main* dock until ``filter_groups_train_batch_size`` prompts are collected.
While the main dock is short the loop generates another batch -- staying in infer mode -- up
to ``filter_groups_max_batches`` times (reference: ``trainer/dapo_trainer_hybrid.py:100-487``).
"""
from __future__ import annotations

import time
from typing import Any, Dict, Iterator, List

import torch

from ..data.transfer_dock import GRPOTransferDock, put_prompts_experience
from ..obs.metrics import Metric, compute_tps, metrics_post_processing, metrics_sort
from ..utils.pad_process import padding_dict_to_tensor_dict
from ..workers.rule_reward import DynamicSampling
from .base import RayBaseTrainer
from .compute_utils import compute_advantage, compute_dapo_data_metrics


class RayDAPOTrainer(RayBaseTrainer):
    def __init__(self, actor_worker, reward_list=None, dynamic_sampling_list=None, **kw):
        super().__init__(actor_worker, None, reward_list, **kw)
        rl = actor_worker.rl_config
        self.should_filter = bool(rl.filter_groups_enable)
        self.max_num_prompt_in_batch = rl.filter_groups_train_batch_size if self.should_filter \
            else self.global_batch_size
        self.max_num_gen_batches = rl.filter_groups_max_batches
        self.dynamic_sampling_list = dynamic_sampling_list
        self.num_gen_batches = 0
        self.num_prompt_in_batch = 0
        self.enable_partial_rollout = self.partial_rollout_max_split > 1
        self.multi_turn_enable = bool(rl.multi_turn_enable)
        self.metrics = Metric()
        self.sampling_metrics = Metric()
        self.transfer_dock = self.sampling_transfer_dock = None
        self.transfer_dock_init()
        gbs_n = self.max_num_prompt_in_batch * self.n_samples_per_prompt
        self.skip_actor_log_prob = (gbs_n == rl.mini_batch_size and rl.epochs == 1)

    def transfer_dock_init(self) -> None:
        cols = self.dataset_additional_keys + ["metric_for_dapo", "response_mask", "tool_call_num"]
        cons = ["dynamic_sampling", "dapo_metrics"]
        # each store is shared right after it is built (the descriptor of the newest one travels)
        main = sampling = None
        # partial rollout lives in the store that the rollout writes: the main store without dynamic sampling,
        # the sampling store with it (the main store then only receives finished, informative groups)
        partial_main = self.enable_partial_rollout and not self.should_filter
        if self.is_driver:
            main = self._new_dock(self.max_num_prompt_in_batch * (2 if partial_main else 1),
                                  self.n_samples_per_prompt, self.metrics,
                                  max_age=self.partial_rollout_max_split if partial_main else 1,
                                  GBS_train=self.max_num_prompt_in_batch, addition_columns=cols,
                                  addition_consumers=cons)
        self.transfer_dock = self._share_dock(main)
        if self.should_filter and self.is_driver:
            two = 2 if self.enable_partial_rollout else 1
            sampling = self._new_dock(self.global_batch_size * two, self.n_samples_per_prompt,
                                      self.sampling_metrics,
                                      max_age=self.partial_rollout_max_split if self.enable_partial_rollout else 1,
                                      GBS_train=self.global_batch_size, addition_columns=cols,
                                      addition_consumers=cons)
        self.sampling_transfer_dock = self._share_dock(sampling) if self.should_filter else None
        self.actor_worker.sync_init_transfer_dock(self.transfer_dock, None, self.sampling_transfer_dock)
        for r in self.reward_list:
            (getattr(r, "sync_init_transfer_dock", None) or r.init_transfer_dock)(
                self.transfer_dock, None, self.sampling_transfer_dock)
        if self.should_filter and self.dynamic_sampling_list is None and self.is_driver:
            self.dynamic_sampling_list = [DynamicSampling(self.actor_worker.rl_config, self.transfer_dock,
                                                          self.sampling_transfer_dock)]
        for d in self.dynamic_sampling_list or []:
            d.init_transfer_dock(self.transfer_dock, None, self.sampling_transfer_dock)

    # ------------------------------------------------------------------------------------------
    def dynamic_sampling(self) -> bool:
        """Move informative groups to the main dock; True = keep generating."""
        self.num_gen_batches += 1
        for d in self.dynamic_sampling_list or []:
            d.dynamic_sampling()
        self.num_prompt_in_batch = self.transfer_dock.get_cur_index() // self.n_samples_per_prompt
        self.logger.info(f"dynamic sampling: {self.num_prompt_in_batch}/{self.max_num_prompt_in_batch} "
                         f"prompt groups after {self.num_gen_batches} generation batch(es)")
        if self.num_prompt_in_batch < self.max_num_prompt_in_batch:
            if self.max_num_gen_batches <= 0 or self.num_gen_batches < self.max_num_gen_batches:
                return True
            raise ValueError("dynamic sampling: generated filter_groups_max_batches batches without "
                             "collecting a full training batch; check the data / reward")
        return False

    def _decide(self, flag: bool) -> bool:
        """Broadcast a driver decision to all ranks."""
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            box = [flag]
            dist.broadcast_object_list(box, src=0)
            return bool(box[0])
        return flag

    def fit(self, data_loader) -> List[Dict[str, Any]]:
        rl = self.actor_worker.rl_config
        td = self.transfer_dock
        gen_td = self.sampling_transfer_dock if self.should_filter else td
        iteration = self.actor_worker.get_iteration()
        n = self.n_samples_per_prompt
        data_iters = iter(data_loader)
        history = []
        all_time = 0.0

        def next_batch():
            nonlocal data_iters
            try:
                return next(data_iters)
            except StopIteration:
                data_iters = iter(data_loader)
                return next(data_iters)

        if self.enable_partial_rollout and self.is_driver:
            # two batches stay in flight: unfinished responses continue beside the fresh prompts
            data, idx = put_prompts_experience(next_batch(), n, self.dataset_additional_keys)
            gen_td.put_experience(padding_dict_to_tensor_dict(data), idx, is_prompt=True)
        while iteration < self.train_iters:
            t0 = time.time()
            if self.is_driver:
                data, idx = put_prompts_experience(next_batch(), n, self.dataset_additional_keys,
                                                   add_another_batch=self.enable_partial_rollout)
                gen_td.put_experience(padding_dict_to_tensor_dict(data), idx, is_prompt=True)
            self._driver_section_done()
            if self.should_filter:
                self.actor_worker.enter_infer_mode(blocking=self.blocking)
            self.actor_worker.generate_sequences(blocking=self.blocking)
            if self.should_filter or self.enable_partial_rollout:
                # the driver is about to judge and clear the sampling store: every rank must have left its
                # rollout loop first (a rank still polling a cleared store would never see it finished); under
                # partial rollout the set of completed groups must stand still before any stage picks its rows
                self.actor_worker.barrier()
            again = False
            for reward in self.reward_list:          # model-based reward scorers: a stage every rank calls
                if hasattr(reward, "worker"):
                    reward.compute_rm_score(blocking=True)
            if self.is_driver:
                for reward in self.reward_list:
                    if not hasattr(reward, "worker"):
                        reward.compute_rm_score()
                if self.should_filter:
                    again = self.dynamic_sampling()
                    # rollout / reward timings were recorded in the sampling dock: carry them over
                    for k, v in list(gen_td.get_metrics().metric.items()):
                        td.update_metrics(k, value=v, cumulate=isinstance(v, list))
                    # under partial rollout only the groups that were judged leave the sampling store; the
                    # unfinished ones stay and are continued beside the next batch of prompts
                    gen_td.clear("dynamic_sampling") if self.enable_partial_rollout else gen_td.clear()
            if self.should_filter:
                if self._decide(again):
                    all_time += time.time() - t0
                    continue
                self.actor_worker.exit_infer_mode(blocking=self.blocking)
            data_num = self.max_num_prompt_in_batch * n
            if self.is_driver:
                t_a = time.time()
                compute_advantage(td, self.gamma, self.lam, self.adv_estimator, rl.adv_dispatch_size,
                                  self.pad_token_id, self.max_num_prompt_in_batch, self.guarantee_order, n,
                                  multi_turn_enable=self.multi_turn_enable)
                t_e = time.time()
                td.update_metrics("timing/adv", value=[round(t_e, 4), round(t_a, 4)], cumulate=True)
                td.update_metrics("end_time/end_adv_time", value=[round(t_e, 4)], cumulate=True)
            self._driver_section_done()
            if not self.skip_actor_log_prob:
                self.actor_worker.compute_log_prob(blocking=self.blocking)
            self.actor_worker.wait_all_ref_objs_run_over()
            self.actor_worker.update(self.kl_ctrl, self.skip_actor_log_prob)
            self._driver_section_done()
            iteration += 1
            if self.is_driver:
                dm = compute_dapo_data_metrics(td, data_num, self.pad_token_id, data_num, self.guarantee_order,
                                               self.multi_turn_enable)
                m = metrics_post_processing(td.get_metrics())
                m.update(dm)
                all_time += time.time() - t0
                m = metrics_sort(m, all_time)
                m["train/num_gen_batches"] = self.num_gen_batches if self.should_filter else 1
                kw = dict(actor_resource=rl.actor_resource, use_integrated_worker=rl.use_integrated_worker)
                m["e2e_tps"] = compute_tps(kw, m, self.max_num_prompt_in_batch, n, all_time, rl.log_max_throughput)
                if m.get("timing/update"):
                    m["update_tps"] = compute_tps(kw, m, self.max_num_prompt_in_batch, n, m["timing/update"],
                                                  rl.log_max_throughput)
                if m.get("timing/rollout"):
                    m["vllm_tps"] = compute_tps(kw, m, self.global_batch_size, n, m["timing/rollout"],
                                                rl.log_max_throughput)
                self.log_metrics(m, iteration, self.train_iters)
                history.append(m)
                td.clear()
            all_time = 0.0
            self.num_gen_batches = self.num_prompt_in_batch = 0
            self._driver_section_done()
            if self.save_interval and (iteration % self.save_interval == 0 or iteration == self.train_iters):
                self.save_checkpoint(iteration)
        return history
