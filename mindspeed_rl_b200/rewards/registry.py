"""Verifier registry and the weighted rule-reward dispatcher.

``compute_verifier_score(batch, rl_config, tokenizer, ...)`` decodes responses / labels, runs
every configured verifier, returns ``(scores [B], per-verifier metrics, raw scores of the metric
used by DAPO filtering)`` and applies the DAPO overlong shaping after the weighted sum
(reference: ``mindspeed_rl/models/rule_verifier.py:81-185``).

Verifiers come in two kinds:
* text verifiers ``f(sequences: list[str], answers: list[str], **kw) -> list[float]``;
* token verifiers ``f(token_rows: list[Tensor], labels, **kw) -> list[float]`` registered with
  ``on_tokens=True`` -- used by the synthetic benchmarks ("response contains token 7").
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

_VERIFIERS: Dict[str, Tuple[Callable, bool]] = {}


def register_verifier(name: str, on_tokens: bool = False):
    def deco(fn):
        _VERIFIERS[name] = (fn, on_tokens)
        return fn
    return deco


def get_verifier(name: str) -> Tuple[Callable, bool]:
    if name not in _VERIFIERS:
        from . import math_verifiers  # noqa: F401  (registers the text verifiers lazily)
    if name not in _VERIFIERS:
        raise ValueError(f"verifier '{name}' is not registered (known: {sorted(_VERIFIERS)})")
    return _VERIFIERS[name]


def known_verifiers() -> List[str]:
    from . import math_verifiers  # noqa: F401
    return sorted(_VERIFIERS)


@register_verifier("contains_token_7", on_tokens=True)
def contains_token_7(token_rows: Sequence[torch.Tensor], labels=None, token_id: int = 7, **_) -> List[float]:
    """1.0 when the response contains ``token_id`` (default 7), else 0.0."""
    return [1.0 if bool((row == token_id).any()) else 0.0 for row in token_rows]


def overlong_penalty(response_length: int, max_tokens: int, buffer: int, factor: float) -> float:
    """DAPO soft overlong punishment: 0 inside ``max_tokens - buffer``, linear down to ``-factor``."""
    if buffer <= 0:
        return 0.0
    expected = max_tokens - buffer
    exceed = response_length - expected
    return min(-min(exceed, buffer) / buffer * factor, 0.0)


def compute_verifier_score(batch: Dict[str, Sequence[torch.Tensor]], rl_config, tokenizer=None,
                           ignore_token: int = -100) -> Tuple[torch.Tensor, Dict[str, List[float]], Optional[List[float]]]:
    """``batch`` holds ragged columns ``responses``, ``response_length`` and optionally ``labels``
    (+ extra dataset keys)."""
    from . import bounded_pool

    bounded_pool.set_parallel(int(getattr(rl_config, "verifier_parallel", 1) or 1))
    responses = [r.reshape(-1) for r in batch["responses"]]
    n = len(responses)
    names: List[str] = list(rl_config.verifier_function)
    weights: List[float] = list(rl_config.verifier_weight)
    texts = answers = None
    total = [0.0] * n
    metrics: Dict[str, List[float]] = {}
    tool_calls = [int(t.reshape(-1)[0]) for t in batch["tool_call_num"]] if "tool_call_num" in batch else None
    for name, w in zip(names, weights):
        fn, on_tokens = get_verifier(name)
        if on_tokens:
            scores = fn(responses, batch.get("labels"))
        else:
            if texts is None:
                if tokenizer is None:
                    raise ValueError(f"verifier '{name}' needs a tokenizer to decode the responses")
                eos = getattr(tokenizer, "eos_token_id", None) or getattr(tokenizer, "eod", 0)

                def dec(row):
                    ids = [eos if int(t) == ignore_token else int(t) for t in row.reshape(-1).tolist()]
                    return tokenizer.decode(ids, skip_special_tokens=True)

                texts = [dec(r) for r in responses]
                answers = [dec(l) for l in batch["labels"]] if "labels" in batch else [""] * n
            scores = fn(texts, answers, tool_call_nums=tool_calls) if tool_calls is not None \
                else fn(texts, answers)
        scores = [float(s) for s in scores]
        metrics[f"{name}_rewards/mean"] = scores
        total = [t + w * s for t, s in zip(total, scores)]
    if getattr(rl_config, "overlong_buffer_enable", False):
        lens = [int(l.reshape(-1)[0]) for l in batch["response_length"]]
        total = [t + overlong_penalty(l, rl_config.rollout_max_tokens, rl_config.overlong_buffer,
                                      rl_config.overlong_buffer_penalty_factor)
                 for t, l in zip(total, lens)]
    filt = getattr(rl_config, "filter_groups_metric", None)
    metric_for_filter = metrics.get(filt) if getattr(rl_config, "filter_groups_enable", False) else None
    return torch.tensor(total, dtype=torch.float32), metrics, metric_for_filter
