"""End-to-end GRPO plumbing on CPU (world size 1, fp32): tiny Qwen2-style decoder, 8 prompts of 64
tokens, 4 samples per prompt, up to 64 new tokens, rule reward "response contains token 7",
group-normalised advantages, clip 0.2, KL 1e-3 to a frozen reference, Adam lr 1e-6, 2 steps."""
import torch

from mindspeed_rl_b200.config import GenerateConfig, MegatronConfig, RLConfig, compose, validate_rl_args
from mindspeed_rl_b200.datasets.synthetic import SyntheticPromptLoader
from mindspeed_rl_b200.runtime.worker_group import SPMDWorkerGroup
from mindspeed_rl_b200.trainer.grpo_trainer import RayGRPOTrainer
from mindspeed_rl_b200.workers.integrated_worker import IntegratedWorker
from mindspeed_rl_b200.workers.rule_reward import RuleReward


def build(n_prompts=8, n_samples=4, max_tokens=64, iters=2):
    model = compose("grpo_tiny_cpu")["model"]
    actor = MegatronConfig(dict(model="tiny_qwen2", global_batch_size=n_prompts, micro_batch_size=4,
                                seq_length=128, lr=1e-6, lr_decay_style="constant", stage="ray_grpo",
                                train_iters=iters, clip_grad=1.0, weight_decay=0.0, seed=0,
                                reset_attention_mask=True), model)
    rl = RLConfig(dict(n_samples_per_prompt=n_samples, mini_batch_size=n_prompts, clip_ratio=0.2,
                       init_kl_coef=0.001, kl_penalty="low_var_kl", adv_estimator="group_norm",
                       verifier_function=["contains_token_7"], verifier_weight=[1.0],
                       actor_resource={"num_gpus": 1}, use_remove_padding=True))
    gen = GenerateConfig(dict(infer_tensor_parallel_size=1, max_num_seqs=64, max_model_len=128,
                              max_num_batched_tokens=1024, kv_block_size=8, enable_prefix_caching=True,
                              sampling_config=dict(max_tokens=max_tokens, temperature=1.0, top_k=-1, top_p=1.0,
                                                   seed=0)))
    validate_rl_args(actor, actor, actor, rl, gen)
    return actor, rl, gen


def test_grpo_two_steps_cpu():
    torch.manual_seed(0)
    actor, rl, gen = build()
    worker = IntegratedWorker(actor, rl, gen, eos_token_id=1023, pad_token_id=0, device="cpu")
    group = SPMDWorkerGroup(worker, num_gpus=1).initialize()
    reward = RuleReward(rl, None, actor)
    trainer = RayGRPOTrainer(group, reward_list=[reward], train_iters=2, save_interval=0,
                             adv_estimator="group_norm", kl_penalty="low_var_kl", init_kl_coef=0.001,
                             global_batch_size=8, n_samples_per_prompt=4, pad_token_id=0)
    before = {k: v.clone() for k, v in worker.model.module.state_dict().items()}
    loader = SyntheticPromptLoader(8, 64, 1024, seed=0)
    history = trainer.fit(iter(loader))
    assert len(history) == 2
    for m in history:
        assert m["response_length/max"] <= 64 and m["prompt_length/mean"] == 64
        assert 0.0 <= m["grpo/score/mean"] <= 1.0
        assert m["e2e_tps"] > 0 and m["timing/rollout"] > 0 and m["timing/update"] > 0
        assert "actor/pg_loss" in m and "actor/kl_loss" in m and "timing/resharding_to_infer" in m
        assert torch.isfinite(torch.tensor(m["actor/grad_norm"]))
    after = worker.model.module.state_dict()
    changed = sum(float((after[k] - before[k]).abs().max()) > 0 for k in before)
    assert changed > 0, "the policy update did not change any parameter"
    # the frozen reference must not move
    ref = worker.ref_model.state_dict()
    assert all(torch.equal(ref[k], before[k]) for k in before)
