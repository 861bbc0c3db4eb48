"""Driver-side stages that work on the experience store only: KL controllers, KL-in-reward,
advantage estimation and per-iteration data metrics.

Each stage follows the common consumer loop -- pull rows that are ready for the stage, compute,
write the new columns back -- against any object with the TransferDock methods (in-process
dock or an RPC proxy).  Numerics: reference ``mindspeed_rl/trainer/utils/compute_utils.py:34-486``
(group-norm in fp64 with unbiased std + 1e-6, GAE reverse scan over the padded width followed by
masked whitening, sparse reward at ``response_length - 1``, adaptive KL controller).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import numpy as np
import torch

from .. import ops
from ..utils.compute import compute_kl_penalty
from ..utils.pad_process import (pad_rows, padding_dict_to_tensor_dict, remove_padding_tensor_dict_to_dict,
                                 truncate_rows)
from ..utils.torch_functional import masked_mean, sequence_mask


class AdaptiveKLController:
    """``beta <- beta * (1 + clip(kl/target - 1, +-0.2) * n / horizon)`` (Ziegler et al.)."""

    def __init__(self, init_kl_coef: float, target_kl: float, horizon: int):
        self.value, self.target, self.horizon = init_kl_coef, target_kl, horizon

    def update(self, current_kl: float, n_steps: int) -> None:
        err = float(np.clip(current_kl / self.target - 1, -0.2, 0.2))
        self.value *= 1 + err * n_steps / self.horizon


class FixedKLController:
    def __init__(self, init_kl_coef: float):
        self.value = init_kl_coef

    def update(self, current_kl: float, n_steps: int) -> None:
        pass


def get_kl_controller(kl_ctrl_type: str, init_kl_coef: float, kl_target: float, kl_horizon: int):
    if kl_ctrl_type == "fixed":
        return FixedKLController(init_kl_coef)
    if kl_ctrl_type == "adaptive":
        if kl_horizon <= 0:
            raise ValueError("adaptive KL control needs a positive horizon")
        return AdaptiveKLController(init_kl_coef, kl_target, kl_horizon)
    raise ValueError(f"unknown kl_ctrl_type '{kl_ctrl_type}'")


def get_current_dp_range_indexes(experience_count: int, assign_batch_size: int,
                                 current_dp_rank: int = 0) -> List[List[int]]:
    """Static row ranges of one consumer: batch ``k`` of this rank covers
    ``[rank*assign + k*count, ...)`` (used when ``guarantee_order`` is set)."""
    start = current_dp_rank * assign_batch_size
    return [list(range(s, s + experience_count))
            for s in range(start, start + assign_batch_size, experience_count)]


def pad_experience(batch: Dict[str, List[torch.Tensor]], pad_id: int = 0, multiple: int = 1
                   ) -> Dict[str, torch.Tensor]:
    """Ragged columns -> padded 2-D tensors (token columns padded with ``pad_id``)."""
    out = {}
    token_cols = ("prompts", "responses", "input_ids", "labels")
    for k, rows in batch.items():
        rows = list(rows)
        if k in token_cols:
            out[k] = pad_rows(rows, pad_id, multiple)
        elif all(r.numel() == 1 for r in rows):
            out[k] = torch.stack([r.reshape(()) for r in rows]).unsqueeze(-1) \
                if k in ("rm_scores", "token_level_rewards") else torch.stack([r.reshape(()) for r in rows])
        else:
            out[k] = pad_rows(rows, 0, multiple)
    return out


def generate_mask(responses: torch.Tensor, response_length: torch.Tensor) -> torch.Tensor:
    return sequence_mask(response_length.reshape(-1), responses.shape[1])


def sparse_reward(scores: torch.Tensor, responses: torch.Tensor, response_length: torch.Tensor
                  ) -> torch.Tensor:
    """Place each sequence score on its last response token."""
    r = torch.zeros_like(responses, dtype=torch.float32)
    last = (response_length.reshape(-1).long() - 1).clamp(min=0)
    r[torch.arange(r.shape[0]), last] = scores.reshape(-1).float()
    return r


def compute_gae_advantage_return(token_level_rewards, values, eos_mask, gamma, lam):
    with torch.no_grad():
        return ops.gae(token_level_rewards, values, eos_mask, float(gamma), float(lam), whiten=True)


def compute_group_norm_advantage_return(token_level_rewards, eos_mask, response_length,
                                        n_sample_per_prompt):
    with torch.no_grad():
        adv = ops.group_norm_advantage(token_level_rewards.reshape(-1), eos_mask, n_sample_per_prompt)
    return adv, adv.clone()


def _consume(td, stage: str, columns: List[str], experience_count: int, sorted_indexes=None,
             get_n_samples: bool = True):
    """Generator over (ragged batch, indexes) until the stage has consumed every row."""
    import time

    while not td.all_consumed(stage):
        idx_arg = sorted_indexes.pop(0) if sorted_indexes else None
        batch, index = td.get_experience(stage, list(columns), experience_count, indexes=idx_arg,
                                         get_n_samples=get_n_samples)
        if not batch or not index:
            time.sleep(0.005)
            continue
        yield remove_padding_tensor_dict_to_dict(batch), index


def apply_kl_penalty(td, experience_count, global_batch_size, guarantee_order, pad_token_id, kl_ctrl,
                     penalty: str = "kl") -> None:
    """``token_level_rewards = sparse(rm_scores) - beta * KL(old || ref)`` (PPO, KL in reward)."""
    columns = ["old_log_prob", "ref_log_prob", "responses", "rm_scores", "response_length"]
    order = get_current_dp_range_indexes(experience_count, global_batch_size) if guarantee_order else None
    for ragged, index in _consume(td, "compute_kl", columns, experience_count, order):
        b = pad_experience(ragged, pad_token_id)
        mask = generate_mask(b["responses"], b["response_length"])
        kld = compute_kl_penalty(b["old_log_prob"], b["ref_log_prob"], penalty) * mask
        rewards = sparse_reward(b["rm_scores"], b["responses"], b["response_length"]) - kl_ctrl.value * kld
        cur = float(masked_mean(kld, mask, axis=-1).mean())
        kl_ctrl.update(current_kl=cur, n_steps=len(index))
        out = {"token_level_rewards": truncate_rows(rewards, b["response_length"])}
        td.put_experience(padding_dict_to_tensor_dict(out), index)


def compute_advantage(td, gamma, lam, adv_estimator, experience_count, pad_token_id, global_batch_size,
                      guarantee_order, n_sample_per_prompt, use_kl_in_reward: bool = False,
                      multi_turn_enable: bool = False) -> None:
    if adv_estimator == "gae":
        columns = ["values", "responses", "token_level_rewards" if use_kl_in_reward else "rm_scores",
                   "response_length"]
    elif adv_estimator == "group_norm":
        columns = ["responses", "rm_scores", "response_length"]
    else:
        raise NotImplementedError(f"adv_estimator '{adv_estimator}'")
    if multi_turn_enable:
        columns.append("response_mask")
    order = get_current_dp_range_indexes(experience_count, global_batch_size) if guarantee_order else None
    for ragged, index in _consume(td, "compute_advantage", columns, experience_count, order):
        b = pad_experience(ragged, pad_token_id)
        mask = b["response_mask"].float() if "response_mask" in b else \
            generate_mask(b["responses"], b["response_length"])
        if adv_estimator == "gae":
            rewards = b["token_level_rewards"] if use_kl_in_reward else \
                sparse_reward(b["rm_scores"], b["responses"], b["response_length"])
            adv, ret = compute_gae_advantage_return(rewards, b["values"], mask, gamma, lam)
        else:
            adv, ret = compute_group_norm_advantage_return(b["rm_scores"], mask, b["response_length"],
                                                           n_sample_per_prompt)
        out = {"advantages": truncate_rows(adv, b["response_length"]),
               "returns": truncate_rows(ret, b["response_length"])}
        td.put_experience(padding_dict_to_tensor_dict(out), index)


def get_last_reward(rm_scores: torch.Tensor, n_sample_batch: int) -> torch.Tensor:
    r = rm_scores.reshape(-1, n_sample_batch)
    return ((r - r.mean(dim=1, keepdim=True)) / (r.std(dim=1, keepdim=True) + 1e-8)).reshape(rm_scores.shape)


def _length_metrics(prefix: str, score: torch.Tensor, resp_len: torch.Tensor, prompt_len: torch.Tensor):
    f = lambda t, how: getattr(t.float() if how == "mean" else t, how)().item()
    out = {}
    for name, t in ((f"{prefix}/score", score), ("response_length", resp_len), ("prompt_length", prompt_len)):
        for how in ("mean", "max", "min"):
            out[f"{name}/{how}"] = f(t, how)
    return out


def compute_grpo_data_metrics(td, experience_count, pad_token_id, global_batch_size, guarantee_order,
                              stage: str = "grpo_metrics", prefix: str = "grpo",
                              multi_turn_enable: bool = False) -> Dict[str, float]:
    columns = ["rm_scores", "responses", "response_length", "prompt_length"]
    if multi_turn_enable:
        columns.append("tool_call_num")
    order = get_current_dp_range_indexes(experience_count, global_batch_size) if guarantee_order else None
    metrics: Dict[str, List[float]] = {}
    for ragged, index in _consume(td, stage, columns, experience_count, order):
        b = pad_experience(ragged, pad_token_id)
        m = _length_metrics(prefix, b["rm_scores"].sum(-1), b["response_length"].reshape(-1),
                            b["prompt_length"].reshape(-1))
        if "tool_call_num" in b:
            t = b["tool_call_num"].reshape(-1)
            m.update({"tool_call_num/mean": t.float().mean().item(), "tool_call_num/max": t.max().item(),
                      "tool_call_num/min": t.min().item()})
        for k, v in m.items():
            metrics.setdefault(k, []).append(v)
    return {k: (max(v) if k.endswith("/max") else min(v) if k.endswith("/min") else sum(v) / len(v))
            for k, v in metrics.items()}


def compute_dapo_data_metrics(td, experience_count, pad_token_id, global_batch_size, guarantee_order,
                              multi_turn_enable: bool = False):
    return compute_grpo_data_metrics(td, experience_count, pad_token_id, global_batch_size,
                                     guarantee_order, "dapo_metrics", "dapo", multi_turn_enable)


def compute_ppo_data_metrics(td, experience_count, pad_token_id, global_batch_size, guarantee_order):
    columns = ["rm_scores", "responses", "response_length", "prompt_length", "advantages", "returns",
               "values"]
    order = get_current_dp_range_indexes(experience_count, global_batch_size) if guarantee_order else None
    metrics: Dict[str, List[float]] = {}
    for ragged, index in _consume(td, "ppo_metrics", columns, experience_count, order):
        b = pad_experience(ragged, pad_token_id)
        mask = generate_mask(b["responses"], b["response_length"])
        m = _length_metrics("critic", b["rm_scores"].sum(-1), b["response_length"].reshape(-1),
                            b["prompt_length"].reshape(-1))
        for name in ("advantages", "returns", "values"):
            t = b[name]
            m[f"critic/{name}/mean"] = masked_mean(t, mask).item()
            m[f"critic/{name}/max"] = t[mask.bool()].max().item()
            m[f"critic/{name}/min"] = t[mask.bool()].min().item()
        for k, v in m.items():
            metrics.setdefault(k, []).append(v)
    return {k: (max(v) if k.endswith("/max") else min(v) if k.endswith("/min") else sum(v) / len(v))
            for k, v in metrics.items()}
