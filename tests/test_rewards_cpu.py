"""Grading under a wall-clock limit: the worker-process pool and the verifiers that use it."""
import math
import time
from types import SimpleNamespace

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
