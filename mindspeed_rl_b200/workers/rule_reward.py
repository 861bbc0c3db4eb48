"""CPU-side reward workers: rule reward and DAPO dynamic sampling.

``RuleReward`` pulls finished rollouts from the experience store, scores them with the
configured verifier set (``rewards.registry``) and writes ``rm_scores`` (plus the raw metric
DAPO filters on).  ``DynamicSampling`` copies prompt groups whose metric is not constant from
the sampling dock into the main dock until the training batch is full.
Reference: ``mindspeed_rl/workers/rule_reward.py:16-159``, ``workers/dynamic_sampling.py:13-102``.
"""
from __future__ import annotations

import time
from typing import List, Optional

import torch

from ..rewards.registry import compute_verifier_score
from ..utils.pad_process import padding_dict_to_tensor_dict, remove_padding_tensor_dict_to_dict


class RuleReward:
    def __init__(self, rl_config=None, tokenizer=None, megatron_config=None, td=None, sampling_td=None):
        self.rl_config = rl_config
        self.tokenizer = tokenizer
        self.megatron_config = megatron_config
        self.td = td
        self.sampling_td = sampling_td
        self.n = rl_config.n_samples_per_prompt if rl_config is not None else 1

    def initialize(self, megatron_config, rl_config, tokenizer, trainer=None):
        self.rl_config, self.megatron_config, self.tokenizer = rl_config, megatron_config, tokenizer
        self.n = rl_config.n_samples_per_prompt

    def init_transfer_dock(self, td, mm_td=None, sampling_transfer_dock=None):
        self.td = td
        self.sampling_td = sampling_transfer_dock

    def compute_rm_score(self) -> None:
        rl = self.rl_config
        dock = self.sampling_td if self.sampling_td is not None else self.td
        columns = ["prompts", "responses", "response_length"]
        extra = list(getattr(self.megatron_config, "dataset_additional_keys", []) or [])
        columns += [k for k in extra if k not in columns]
        if rl.multi_turn_enable:
            columns.append("tool_call_num")
        start = time.time()
        while not dock.all_consumed("rule_reward"):
            batch, idx = dock.get_experience("rule_reward", list(columns), rl.reward_dispatch_size,
                                             get_n_samples=True)
            if not batch or not idx:
                time.sleep(0.002)
                continue
            ragged = remove_padding_tensor_dict_to_dict(batch)
            scores, metrics, filt = compute_verifier_score(ragged, rl, self.tokenizer)
            out = {"rm_scores": [s.reshape(1) for s in scores]}
            if filt is not None:
                out["metric_for_dapo"] = [torch.tensor([v], dtype=torch.float32) for v in filt]
            dock.put_experience(padding_dict_to_tensor_dict(out), idx)
            for k, v in metrics.items():
                dock.update_metrics(k, value=[sum(v) / max(len(v), 1)], cumulate=True)
        end = time.time()
        dock.update_metrics("timing/rule_reward", value=[round(end, 4), round(start, 4)], cumulate=True)
        dock.update_metrics("start_time/rule_reward", value=[round(start, 4)], cumulate=True)
        dock.update_metrics("end_time/rule_reward", value=[round(end, 4)], cumulate=True)


class DynamicSampling:
    """Keep prompt groups with ``std(metric) > 0`` (neither all right nor all wrong)."""

    def __init__(self, rl_config=None, td=None, sampling_td=None):
        self.rl_config, self.td, self.sampling_td = rl_config, td, sampling_td

    def initialize(self, megatron_config, rl_config, tokenizer=None):
        self.rl_config = rl_config

    def init_transfer_dock(self, td, mm_td=None, sampling_transfer_dock=None):
        self.td, self.sampling_td = td, sampling_transfer_dock

    def dynamic_sampling(self) -> int:
        """Returns the number of prompt groups moved into the main dock by this call."""
        rl = self.rl_config
        n = rl.n_samples_per_prompt
        columns = ["prompts", "prompt_length", "responses", "response_length", "input_ids", "rm_scores",
                   "metric_for_dapo"]
        moved = 0
        src, dst = self.sampling_td, self.td
        while not src.all_consumed("dynamic_sampling"):
            batch, idx = src.get_experience("dynamic_sampling", list(columns),
                                            rl.dynamic_sampling_dispatch_size, get_n_samples=True)
            if not batch or not idx:
                time.sleep(0.002)
                continue
            ragged = remove_padding_tensor_dict_to_dict(batch)
            metric = torch.stack([m.reshape(()) for m in ragged["metric_for_dapo"]]).view(-1, n)
            keep_groups = (metric.std(dim=-1) > 0).nonzero(as_tuple=True)[0].tolist()
            for g in keep_groups:
                if dst.get_cur_index() >= rl.filter_groups_train_batch_size * n:
                    break
                target = dst.prefetch_request_index(n)
                if not target:
                    break
                rows = list(range(g * n, (g + 1) * n))[:len(target)]
                out = {k: [ragged[k][r] for r in rows] for k in columns}
                dst.put_experience(padding_dict_to_tensor_dict(out), target)
                moved += 1
        return moved
