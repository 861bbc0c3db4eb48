"""Text verifiers (format / step / accuracy families) registered under the names the YAML
``verifier_function`` list uses (reference table: ``mindspeed_rl/models/rule_verifier.py:188-519``,
``mindspeed_rl/models/math_dapo.py:6-274``).  Accuracy verifiers grade with
``rewards.math_grader``; every call that may run sympy is bounded by a timeout."""
from __future__ import annotations

import re
from typing import List, Optional, Sequence

from .registry import register_verifier
from . import math_grader as G

_FORMAT_RE = re.compile(r"^<think>.*?</think>\s*<answer>.*?</answer>$", re.DOTALL | re.MULTILINE)
_BASE_RE = re.compile(r"^<think>.*?</think>.*?<answer>.*?\\boxed\{.*?\}.*?</answer>$", re.DOTALL)
_STEP_RE = re.compile(r"(Step \d+:|^\d+\.|\n-|\n\*|First,|Second,|Next,|Finally,)", re.MULTILINE)
_STOP_WORDS = ("</s>", "<|im_end|>", "<|endoftext|>")
_ASSISTANT = "<|im_start|>assistant\n"


def _strip_to_answer(text: str) -> str:
    if _ASSISTANT in text:
        text = text.split(_ASSISTANT, 1)[1]
    for w in _STOP_WORDS:
        if w in text:
            text = text.split(w, 1)[0]
    return text.strip()


@register_verifier("format")
def format_reward(sequences: Sequence[str], answers=None, **_) -> List[float]:
    return [1.0 if _FORMAT_RE.match(s.strip()) else 0.0 for s in sequences]


@register_verifier("step")
def reasoning_steps_reward(sequences: Sequence[str], answers=None, **_) -> List[float]:
    return [min(1.0, len(_STEP_RE.findall(s)) / 3) for s in sequences]


def _strict_format_ok(s: str) -> bool:
    s = s.strip()
    if not (s.startswith("<think>") and s.endswith("</answer>")):
        return False
    order = ["<think>", "</think>", "<answer>", "\\boxed{", "</answer>"]
    pos = -1
    for tag in order:
        if s.count(tag) != 1:
            return False
        nxt = s.find(tag)
        if nxt < pos:
            return False
        pos = nxt
    return True


@register_verifier("strict_format")
def strict_format_reward(sequences: Sequence[str], answers=None, **_) -> List[float]:
    oks = G.bounded_map(_strict_format_ok, [(s,) for s in sequences], timeout=1.0, default=None)
    return [0.0 if ok is None else (1.0 if ok else -0.5) for ok in oks]


@register_verifier("acc")
def accuracy_reward(sequences: Sequence[str], answers: Sequence[str], **_) -> List[float]:
    """+1 correct, -0.5 boxed but wrong, -1 no boxed answer, 0 on timeout."""
    out: List[float] = [-1.0] * len(sequences)
    graded, pairs = [], []
    for i, (s, a) in enumerate(zip(sequences, answers)):
        body = _strip_to_answer(s)
        if "boxed" not in body:
            continue
        pred = G.extract_answer(body)
        if pred is None or pred == "":
            continue
        graded.append(i)
        pairs.append((pred, a))
    for i, ok in zip(graded, G.bounded_map(G.math_equal, pairs, timeout=1.0, default=None)):
        out[i] = 0.0 if ok is None else (1.0 if ok else -0.5)
    return out


@register_verifier("base_acc")
def base_model_accuracy_reward(sequences: Sequence[str], answers: Sequence[str], **_) -> List[float]:
    out = []
    for s, a in zip(sequences, answers):
        if not _BASE_RE.match(s.strip()):
            out.append(0.0)
            continue
        boxed = G.extract_boxed_content(s)
        out.append(1.0 if boxed is not None and G.grade_answer(boxed, a) else 0.0)
    return out


def warm_up() -> None:
    G.warm_up()


def _boxed_correct(s: str, a: str) -> bool:
    boxed = G.extract_boxed_content(s)
    return boxed is not None and G.grade_answer(boxed, a)


def _boxed_grade(sequences, answers) -> List[float]:
    # grade_answer bounds its own symbolic step at 2 s; the outer limit only matters for worker processes
    oks = G.bounded_map(_boxed_correct, list(zip(sequences, answers)), timeout=3.0, default=False)
    return [1.0 if ok else 0.0 for ok in oks]


@register_verifier("math_17k_acc")
def math_17k_accuracy_reward(sequences, answers, **_):
    return _boxed_grade(sequences, answers)


@register_verifier("acc_for_ppo")
def ppo_accuracy_reward(sequences, answers, **_):
    return _boxed_grade(sequences, answers)


@register_verifier("math_verify_reward")
def math_verify_reward(sequences, answers, **_):
    out = []
    for s, a in zip(sequences, answers):
        if not _FORMAT_RE.match(s.strip()) and "\\boxed" not in s:
            out.append(0.0)
            continue
        out.append(G.math_verify_score(s, a))
    return out


@register_verifier("acc_for_dapo")
def dapo_accuracy_reward(sequences, answers, **_):
    """+1 / -1 on the last ``Answer:`` line within the final 300 characters (Minerva normalisation)."""
    return [1.0 if G.dapo_is_correct(s[-300:], a) else -1.0 for s, a in zip(sequences, answers)]


@register_verifier("retool_reward")
def retool_reward(sequences, answers, tool_call_nums: Optional[Sequence[int]] = None, **_):
    out = []
    for i, (s, a) in enumerate(zip(sequences, answers)):
        if G.dapo_is_correct_boxed(s[-100:], a):
            out.append(1.0)
        else:
            calls = tool_call_nums[i] if tool_call_nums is not None else 0
            out.append(min(0.0, -1.0 + 0.1 * calls))
    return out
