"""Grading under a wall-clock limit: the worker-process pool and the verifiers that use it."""
import math
import time
from types import SimpleNamespace

import pytest
import torch

from mindspeed_rl_b200.rewards import bounded_pool
from mindspeed_rl_b200.rewards import math_grader as G
from mindspeed_rl_b200.rewards.registry import compute_verifier_score, get_verifier


def test_pool_keeps_order_and_ends_calls_that_pass_their_limit():
    pool = bounded_pool.BoundedPool(workers=2)
    try:
        vals = pool.map(math.sqrt, [(float(i * i),) for i in range(9)], timeout=5.0, default=-1.0)
        assert vals == [float(i) for i in range(9)]
        t0 = time.monotonic()
        # the sleeping call is cut off, its worker replaced, and the calls queued behind it still run
        got = pool.map(time.sleep, [(0.01,), (30.0,), (0.01,), (0.01,)], timeout=0.5, default="late")
        assert got == [None, "late", None, None]
        assert time.monotonic() - t0 < 10.0
        assert pool.timeouts == 1 and pool.restarts == 1
        # a call that raises yields the default and keeps its worker
        assert pool.map(math.sqrt, [(-1.0,), (4.0,)], timeout=5.0, default="bad") == ["bad", 2.0]
        assert pool.restarts == 1
        # a limit on the whole batch
        got = pool.map(time.sleep, [(30.0,), (30.0,), (30.0,)], timeout=20.0, default="late", total_timeout=0.5)
        assert got == ["late"] * 3
        assert pool.map(math.sqrt, [(9.0,)], timeout=5.0) == [3.0]
    finally:
        pool.close()


def test_verifiers_score_the_same_in_worker_processes():
    seqs = ["<think>a</think><answer>so \\boxed{\\frac{1}{2}}</answer>", "the answer is \\boxed{3}", "no box at all",
            "<think>b</think><answer>\\boxed{7}</answer>"]
    answers = ["0.5", "4", "1", "7"]
    names = ["acc", "strict_format", "math_17k_acc", "acc_for_ppo"]
    try:
        bounded_pool.set_parallel(1)
        here = {n: get_verifier(n)[0](seqs, answers) for n in names}
        bounded_pool.set_parallel(2)
        there = {n: get_verifier(n)[0](seqs, answers) for n in names}
        assert bounded_pool.shared_pool().workers, "the pool was not used"
    finally:
        bounded_pool.set_parallel(1)
    assert here == there
    assert here["acc"] == [1.0, -0.5, -1.0, 1.0]
    assert here["math_17k_acc"] == [1.0, 0.0, 0.0, 1.0]


def test_verifier_parallel_is_taken_from_the_config():
    class Tok:
        eos_token_id = 0

        def decode(self, ids, skip_special_tokens=True):
            return "\\boxed{" + str(ids[0]) + "}" if len(ids) == 1 else str(ids[0])

    cfg = SimpleNamespace(verifier_function=["math_17k_acc"], verifier_weight=[1.0], verifier_parallel=2)
    batch = {"responses": [torch.tensor([5]), torch.tensor([6])], "response_length": [torch.tensor([1])] * 2,
             "labels": [torch.tensor([5, 0]), torch.tensor([7, 0])]}
    try:
        scores, metrics, _ = compute_verifier_score(batch, cfg, Tok())
        assert bounded_pool.parallel() == 2
    finally:
        bounded_pool.set_parallel(1)
    assert scores.tolist() == [1.0, 0.0] and metrics["math_17k_acc_rewards/mean"] == [1.0, 0.0]


def test_bounded_map_in_process_fallback():
    assert G.bounded_map(math.sqrt, [(4.0,), (-1.0,)], timeout=1.0, default=None) == [2.0, None]


def test_verifier_score_table():
    """Score values of every rule verifier on hand-made responses."""
    def run(name, seqs, answers, **kw):
        return get_verifier(name)[0](seqs, answers, **kw)

    good = "<think>work</think><answer>so \\boxed{12}</answer>"
    assert run("format", [good, "<think>x</think> no answer tag"], ["", ""]) == [1.0, 0.0]
    assert run("strict_format", [good, "<think>a</think><think>b</think><answer>\\boxed{1}</answer>", "text"],
               ["", "", ""]) == [1.0, -0.5, -0.5]
    steps = "Step 1: a\nStep 2: b\nFirst, c\nFinally, d"
    assert run("step", [steps, "Step 1: only", "nothing"], ["", "", ""]) == [1.0, pytest.approx(1 / 3), 0.0]
    assert run("base_acc", [good, good, "\\boxed{12}"], ["12", "13", "12"]) == [1.0, 0.0, 0.0]
    assert run("acc", ["answer \\boxed{12}", "answer \\boxed{11}", "answer 12"], ["12", "12", "12"]) == [1.0, -0.5, -1.0]
    assert run("acc_for_dapo", ["reasoning\nAnswer: $12$", "Answer: 13", "no marker 12"], ["12", "12", "12"]) == [1.0, -1.0, -1.0]
    # an early "Answer:" outside the last 300 characters does not count
    assert run("acc_for_dapo", ["Answer: 12\n" + "x" * 400], ["12"]) == [-1.0]
    assert run("retool_reward", ["... \\boxed{12}", "... \\boxed{7}", "... \\boxed{7}", "none"], ["12", "12", "12", "12"],
               tool_call_nums=[0, 3, 30, 0]) == [1.0, pytest.approx(-0.7), 0.0, -1.0]
    assert run("math_verify_reward", [good, "plain text 12"], ["12", "12"]) == [1.0, 0.0]
    assert run("math_17k_acc", ["\\boxed{\\frac{1}{2}}", "\\boxed{0.5}", "\\boxed{50\\%}", "0.5"], ["0.5"] * 4) == [1.0, 1.0, 1.0, 0.0]


def test_math_grader_equivalences():
    eq = G.math_equal
    assert eq("1,000", "1000") and eq("0.5", "\\frac{1}{2}") and eq("50%", "0.5") and eq("50", "0.5")
    assert not eq("50", "0.5", include_percentage=False)
    assert eq("(1, 2)", "(1,2)") and not eq("(1, 2)", "[1, 2]") and not eq("(1, 2)", "(1, 2, 3)")
    assert eq("(0.5, x)", "(\\frac{1}{2}, x)")
    assert eq("x = 5", "5") and not eq("x = 5", "6")
    assert eq("2*x + 2", "2*(x + 1)") and not eq("2*x + 2", "2*x + 3")              # symbolic
    assert eq("x + y = 2*z", "2*z - y = x")                                            # equations, sides moved
    assert not eq(None, "1") and not eq("1", None)
    assert G.symbolic_equal("x**2 - 1", "(x - 1)*(x + 1)") and not G.symbolic_equal("x +", "x")
    assert G._split_elements("(a,(b,c),d)") == ["a", "(b,c)", "d"] and G._split_elements("a,b") is None
    assert G.grade_answer(None, "1") is False and G.grade_answer("3", "3.0")
    assert G.extract_boxed_content("a \\boxed{1} then \\boxed{\\frac{3}{4}}") == "\\frac{3}{4}"
    assert G.extract_boxed_content("no box") is None and G.last_boxed_span("\\boxed{unclosed") is None
    assert G.normalize_final_answer("$3$ dollars") == "3" and G.normalize_final_answer("x = \\text{12} cm") == "12"
    assert G.dapo_is_correct("Answer: 1,234", "1234") and not G.dapo_is_correct("the result is 5", "5")
    assert G.dapo_is_correct_boxed("so \\boxed{\\text{7}}", "7") and not G.dapo_is_correct_boxed("7", "7")
    assert G.math_verify_score("\\boxed{4}", "4") == 1.0 and G.math_verify_score("\\boxed{5}", "4") == 0.0


def test_overlong_penalty_values():
    from mindspeed_rl_b200.rewards.registry import overlong_penalty
    assert overlong_penalty(100, 200, 50, 1.0) == 0.0              # inside max_tokens - buffer
    assert overlong_penalty(175, 200, 50, 1.0) == pytest.approx(-0.5)
    assert overlong_penalty(400, 200, 50, 2.0) == pytest.approx(-2.0)
    assert overlong_penalty(400, 200, 0, 2.0) == 0.0
