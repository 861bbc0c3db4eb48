"""Numeric regression of a tiny GRPO run against stored values (relative 2 % / absolute 0.01, the
tolerances of the reference's system tests that compare entropy / pg_loss / grad_norm / response
length with ``baseline_results/*.json``).  Regenerate the file on purpose with
``MSRL_UPDATE_BASELINE=1 python -m pytest tests/test_regression_cpu.py``."""
import json
import os
from pathlib import Path

import torch

from test_e2e_grpo_cpu import build
from mindspeed_rl_b200.datasets.synthetic import SyntheticPromptLoader
from mindspeed_rl_b200.runtime.worker_group import SPMDWorkerGroup
from mindspeed_rl_b200.trainer.grpo_trainer import RayGRPOTrainer
from mindspeed_rl_b200.workers.integrated_worker import IntegratedWorker
from mindspeed_rl_b200.workers.rule_reward import RuleReward

BASELINE = Path(__file__).parent / "baseline_results" / "grpo_tiny_cpu.json"
KEYS = ["actor/entropy", "actor/pg_loss", "actor/kl_loss", "actor/grad_norm", "grpo/score/mean",
        "response_length/mean", "response_length/max"]


def _run():
    torch.manual_seed(0)
    torch.set_num_threads(1)                     # a fixed reduction order on every machine
    actor, rl, gen = build()
    worker = IntegratedWorker(actor, rl, gen, eos_token_id=1023, pad_token_id=0, device="cpu")
    group = SPMDWorkerGroup(worker, num_gpus=1).initialize()
    trainer = RayGRPOTrainer(group, reward_list=[RuleReward(rl, None, actor)], train_iters=2, save_interval=0,
                             adv_estimator="group_norm", kl_penalty="low_var_kl", init_kl_coef=0.001,
                             global_batch_size=8, n_samples_per_prompt=4, pad_token_id=0)
    history = trainer.fit(iter(SyntheticPromptLoader(8, 64, 1024, seed=0)))
    return [{k: float(m[k]) for k in KEYS if k in m} for m in history]


def test_tiny_grpo_matches_the_stored_baseline():
    threads = torch.get_num_threads()
    try:
        got = _run()
    finally:
        torch.set_num_threads(threads)
    if os.environ.get("MSRL_UPDATE_BASELINE") == "1" or not BASELINE.exists():
        BASELINE.write_text(json.dumps(got, indent=1))
    want = json.loads(BASELINE.read_text())
    assert len(got) == len(want)
    for step, (g, w) in enumerate(zip(got, want)):
        assert set(g) == set(w)
        for k in w:
            assert abs(g[k] - w[k]) <= max(0.02 * abs(w[k]), 0.01), (step, k, g[k], w[k])
