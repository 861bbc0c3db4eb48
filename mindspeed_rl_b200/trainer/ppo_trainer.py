"""PPO driver loop (actor + critic + frozen reference, GAE advantages).

Order of one iteration (reference: ``mindspeed_rl/trainer/ppo_trainer_hybrid.py:180-237``):
rollout -> reference log-probs -> old log-probs -> critic values -> reward -> optional KL-in-reward
-> GAE advantages -> critic update -> actor update -> metrics.
"""
from __future__ import annotations

import time
from typing import Any, Dict, Iterator, List

import torch

from ..data.transfer_dock import GRPOTransferDock, put_prompts_experience
from ..obs.metrics import Metric, compute_tps, metrics_post_processing, metrics_sort
from ..utils.pad_process import padding_dict_to_tensor_dict
from .base import RayBaseTrainer
from .compute_utils import apply_kl_penalty, compute_advantage, compute_ppo_data_metrics


class RayPPOTrainer(RayBaseTrainer):
    def __init__(self, actor_worker, ref_worker=None, reward_list=None, critic_worker=None, **kw):
        kw.setdefault("adv_estimator", "gae")
        super().__init__(actor_worker, ref_worker or actor_worker, reward_list, critic_worker, **kw)
        self.metrics = Metric()
        self.transfer_dock = None
        self.transfer_dock_init()
        self.skip_actor_log_prob = False

    def transfer_dock_init(self) -> None:
        dock = None
        cols = self.dataset_additional_keys + ["values"]
        if getattr(getattr(self.actor_worker, "rl_config", None), "multi_turn_enable", False):
            cols += ["response_mask", "tool_call_num"]          # written by the multi-turn rollout loop
        if self.is_driver:
            dock = self._new_dock(
                self.global_batch_size, self.n_samples_per_prompt, self.metrics,
                addition_columns=cols,
                addition_consumers=["compute_kl", "critic_train", "critic_compute_values", "ppo_metrics"])
        self.transfer_dock = self._share_dock(dock)
        for w in {id(x): x for x in (self.actor_worker, self.ref_worker, self.critic_worker) if x is not None}.values():
            w.sync_init_transfer_dock(self.transfer_dock)
        for r in self.reward_list:
            (getattr(r, "sync_init_transfer_dock", None) or r.init_transfer_dock)(self.transfer_dock)

    def fit(self, data_iters: Iterator[Dict[str, List[torch.Tensor]]]) -> List[Dict[str, Any]]:
        rl = self.actor_worker.rl_config
        td = self.transfer_dock
        iteration = self.actor_worker.get_iteration()
        n, gbs = self.n_samples_per_prompt, self.global_batch_size
        history = []
        while iteration < self.train_iters:
            t0 = time.time()
            if self.is_driver:
                batch = next(data_iters)
                data, idx = put_prompts_experience(batch, n, self.dataset_additional_keys)
                td.put_experience(padding_dict_to_tensor_dict(data), idx, is_prompt=True)
            self._driver_section_done()
            self.actor_worker.generate_sequences(blocking=self.blocking)
            self.ref_worker.compute_ref_log_prob(blocking=self.blocking)
            self.actor_worker.compute_log_prob(blocking=self.blocking)
            self.critic_worker.compute_values(blocking=self.blocking)
            for reward in self.reward_list:      # model-based reward workers are SPMD stages
                if hasattr(reward, "worker"):
                    reward.compute_rm_score(blocking=self.blocking)
            if self.is_driver:
                for reward in self.reward_list:
                    if not hasattr(reward, "worker"):
                        reward.compute_rm_score()
                if self.use_kl_in_reward:
                    t_k = time.time()
                    apply_kl_penalty(td, rl.kl_dispatch_size or gbs * n, gbs, self.guarantee_order,
                                     self.pad_token_id, self.kl_ctrl, self.kl_penalty)
                    td.update_metrics("timing/kl", value=[round(time.time(), 4), round(t_k, 4)], cumulate=True)
                t_a = time.time()
                compute_advantage(td, self.gamma, self.lam, self.adv_estimator, rl.adv_dispatch_size,
                                  self.pad_token_id, gbs, self.guarantee_order, n,
                                  use_kl_in_reward=self.use_kl_in_reward, multi_turn_enable=rl.multi_turn_enable)
                t_e = time.time()
                td.update_metrics("timing/adv", value=[round(t_e, 4), round(t_a, 4)], cumulate=True)
                td.update_metrics("end_time/end_adv_time", value=[round(t_e, 4)], cumulate=True)
            self._driver_section_done()
            self.critic_worker.update_critic(blocking=self.blocking)
            self.actor_worker.update(self.kl_ctrl, self.skip_actor_log_prob)
            self._driver_section_done()
            iteration += 1
            if self.is_driver:
                dm = compute_ppo_data_metrics(td, gbs * n, self.pad_token_id, gbs, self.guarantee_order)
                m = metrics_post_processing(td.get_metrics())
                m.update(dm)
                time_all = time.time() - t0
                m = metrics_sort(m, time_all)
                kw = dict(actor_resource=rl.actor_resource, reference_resource=rl.reference_resource,
                          reward_resource=rl.reward_resource, use_integrated_worker=rl.use_integrated_worker)
                m["e2e_tps"] = compute_tps(kw, m, gbs, n, time_all, rl.log_max_throughput)
                if m.get("timing/update"):
                    m["update_tps"] = compute_tps(kw, m, gbs, n, m["timing/update"], rl.log_max_throughput)
                if m.get("timing/rollout"):
                    m["vllm_tps"] = compute_tps(kw, m, gbs, n, m["timing/rollout"], rl.log_max_throughput)
                self.log_metrics(m, iteration, self.train_iters)
                history.append(m)
                td.clear()
            self._driver_section_done()
            if self.save_interval and (iteration % self.save_interval == 0 or iteration == self.train_iters):
                self.save_checkpoint(iteration)
        return history
