"""Metric accumulation and the per-iteration post-processing (timings, throughput).

* ``Metric`` lives inside the experience store; workers push values with
  ``update(key, value, cumulate=True)``.
* Timing keys carry wall-clock stamps ``[end, start]`` from every rank, so the iteration value
  is ``max(all) - min(all)``; ``timing/resharding_*`` entries are durations and take the max.
* ``compute_tps`` is the headline throughput:
  ``(prompt_len + response_len) * global_batch * n_samples / n_devices / seconds``.

Reference definitions: ``mindspeed_rl/utils/metrics.py:10-141``,
``mindspeed_rl/utils/utils.py:195-303``.
"""
from __future__ import annotations

from numbers import Number
from typing import Any, Dict, Iterable, List, Optional

import numpy as np
import torch


def _numbers(values: Iterable[Any]) -> List[float]:
    return [float(v) for v in values if isinstance(v, Number) and not isinstance(v, bool)]


def _reduce(value: Any, how: str):
    if isinstance(value, torch.Tensor):
        v = value.detach().float()
        return {"mean": v.mean, "sum": v.sum, "max": v.max, "min": v.min}[how]().item()
    if isinstance(value, np.ndarray):
        return {"mean": np.mean, "sum": np.sum, "max": np.max, "min": np.min}[how](value, axis=0)
    if isinstance(value, dict):
        value = list(value.values())
    if isinstance(value, (list, tuple)):
        nums = _numbers(value)
        if not nums:
            return None
        if how == "mean":
            return sum(nums) / len(nums)
        return {"sum": sum, "max": max, "min": min}[how](nums)
    return None


class Metric:
    def __init__(self):
        self.metric: Dict[str, Any] = {}

    def update(self, key: str = "", value: Any = None, cumulate: bool = False) -> None:
        """Set ``metric[key] = value`` or, with ``cumulate``, extend the list stored under it.
        A dict ``value`` updates/extends every key it contains."""
        items = value.items() if isinstance(value, dict) else [(key, value)]
        for k, v in items:
            if not cumulate:
                self.metric[k] = v
                continue
            seq = list(v) if isinstance(v, (list, tuple)) else [v]
            cur = self.metric.get(k)
            if isinstance(cur, list):
                cur.extend(seq)
            else:
                self.metric[k] = seq

    def compute_mean(self, key, value, axis=0):
        return _reduce(value, "mean")

    def compute_sum(self, value, axis=0):
        return _reduce(value, "sum")

    def compute_max(self, key, value, axis=0):
        return _reduce(value, "max")

    def compute_min(self, key, value, axis=0):
        return _reduce(value, "min")

    def remove_key(self, key: str) -> None:
        self.metric.pop(key, None)

    def reset(self) -> None:
        self.metric = {}

    def keys(self):
        return self.metric.keys()


def metrics_post_processing(metrics: Metric) -> Dict[str, Any]:
    out: Dict[str, Any] = {}
    for key, value in metrics.metric.items():
        is_list = isinstance(value, list)
        if not is_list:
            out[key] = value
        elif "timing" in key:
            if "resharding" in key:
                out[key] = metrics.compute_max(key, value)
            else:
                out[key] = metrics.compute_max(key, value) - metrics.compute_min(key, value)
        elif "start_time" in key:
            out[key] = metrics.compute_min(key, value)
        elif "end_time" in key:
            out[key] = metrics.compute_max(key, value)
        else:
            out[key] = metrics.compute_mean(key, value)
    return out


_HEAD_ORDER = ["timing/all", "timing/update", "timing/rollout", "timing/old_log_p",
               "timing/reference_model", "timing/resharding_to_infer", "timing/resharding_to_train",
               "timing/adv", "timing/non_overlap_reference_model"]
_SECOND_ORDER = ["timing/non_overlap_rule_reward", "timing/non_overlap_reward_model",
                 "timing/non_overlap_adv", "timing/rule_reward", "timing/reward_model",
                 "timing/ref_onload", "timing/ref_offload", "timing/critic_model",
                 "timing/update_critic"]


def metrics_sort(metrics: Dict[str, Any], time_all: float) -> Dict[str, Any]:
    """Derive the non-overlapped stage times and put the timing keys first."""
    m = dict(metrics)
    old_end = m.pop("end_time/old_log_p", None)
    adv_end = m.pop("end_time/end_adv_time", None)
    ref_start = m.pop("start_time/reference_model", None)
    ref_end = m.pop("end_time/reference", None)
    head = list(_HEAD_ORDER)
    has_ref, has_old = ref_end is not None, old_end is not None
    if not has_ref:
        head.remove("timing/reference_model")
        head.remove("timing/non_overlap_reference_model")
        ref_end = 0
    if not has_old:
        old_end = ref_end
        head.remove("timing/old_log_p")
    if ref_start is None:
        ref_start = 0
    m_ref = max(ref_end - max(old_end, ref_start), 0) if has_ref else 0
    if not has_old and not has_ref:
        m_adv = m.get("timing/adv", 0)
    else:
        m_adv = max((adv_end or 0) - old_end, 0)
    for name in ("rule_reward", "reward_model"):
        if f"timing/{name}" in m:
            st, en = m.pop(f"start_time/{name}", None), m.pop(f"end_time/{name}", None)
            if st is not None and en is not None:
                m[f"timing/non_overlap_{name}"] = max(en - max(old_end, st), 0)
    m["timing/non_overlap_reference_model"] = m_ref
    m["timing/non_overlap_adv"] = m_adv
    m["timing/all"] = time_all
    ordered = dict(sorted(m.items()))
    second = [k for k in ordered if k in _SECOND_ORDER]
    rest = [k for k in ordered if k not in head and k not in _SECOND_ORDER]
    return {k: ordered[k] for k in head + second + rest if k in ordered}


def compute_tps(compute_kwargs: Dict[str, Any], metrics_result: Dict[str, Any], gbs: int,
                n_samples: int, time_all: float, log_max_throughput: bool = False) -> float:
    def gpus(res):
        if not res:
            return 0
        return res.get("num_npus", res.get("num_gpus", 0)) or 0

    actor = gpus(compute_kwargs.get("actor_resource"))
    if compute_kwargs.get("use_integrated_worker", False):
        world = actor
    else:
        world = actor + gpus(compute_kwargs.get("reference_resource")) + gpus(compute_kwargs.get("reward_resource"))
    kind = "max" if log_max_throughput else "mean"
    tokens = metrics_result[f"response_length/{kind}"] + metrics_result[f"prompt_length/{kind}"]
    return tokens * gbs * n_samples / max(world, 1) / time_all
