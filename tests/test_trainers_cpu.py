"""DAPO (dynamic sampling, clip-higher, overlong shaping) and PPO (critic, GAE, KL in reward) driver
loops end to end on CPU with the tiny decoder."""
import torch

from mindspeed_rl_b200.config import GenerateConfig, MegatronConfig, RLConfig, validate_rl_args
from mindspeed_rl_b200.config.loader import load_model_catalogue
from mindspeed_rl_b200.datasets.synthetic import SyntheticPromptLoader
from mindspeed_rl_b200.runtime.worker_group import SPMDWorkerGroup
from mindspeed_rl_b200.trainer.dapo_trainer import RayDAPOTrainer
from mindspeed_rl_b200.trainer.ppo_trainer import RayPPOTrainer
from mindspeed_rl_b200.workers.integrated_worker import IntegratedWorker
from mindspeed_rl_b200.workers.model_workers import CriticWorker
from mindspeed_rl_b200.workers.rule_reward import RuleReward


def _configs(stage, vocab=64, **rl_extra):
    cat = load_model_catalogue(["tiny_qwen2"])
    cat["tiny_qwen2"].update(padded_vocab_size=vocab, hidden_size=64, ffn_hidden_size=128, num_layers=2)
    actor = MegatronConfig(dict(model="tiny_qwen2", global_batch_size=4, micro_batch_size=4, seq_length=64,
                                lr=1e-4, lr_decay_style="constant", stage=stage, train_iters=2, clip_grad=1.0,
                                weight_decay=0.0, seed=0, reset_attention_mask=True), cat)
    rl = RLConfig(dict(n_samples_per_prompt=4, mini_batch_size=4, verifier_function=["contains_token_7"],
                       verifier_weight=[1.0], actor_resource={"num_gpus": 1}, use_remove_padding=True, **rl_extra))
    gen = GenerateConfig(dict(infer_tensor_parallel_size=1, max_num_seqs=32, max_model_len=64,
                              max_num_batched_tokens=512, kv_block_size=8,
                              sampling_config=dict(max_tokens=16, temperature=1.0, top_k=-1, top_p=1.0, seed=1)))
    return actor, rl, gen


def test_dapo_dynamic_sampling_cpu():
    torch.manual_seed(0)
    actor, rl, gen = _configs("ray_dapo", clip_higher_enable=True, clip_ratio_low=0.2, clip_ratio_high=0.28,
                              filter_groups_enable=True, filter_groups_metric="contains_token_7",
                              filter_groups_max_batches=20, filter_groups_train_batch_size=2,
                              overlong_buffer_enable=True, overlong_buffer=4, rollout_max_tokens=16,
                              token_level_loss=True)
    validate_rl_args(actor, None, actor, rl, gen)
    assert rl.filter_groups_metric == "contains_token_7_rewards/mean"
    worker = IntegratedWorker(actor, rl, gen, eos_token_id=63, pad_token_id=0, device="cpu", with_reference=False)
    group = SPMDWorkerGroup(worker, 1).initialize()
    trainer = RayDAPOTrainer(group, reward_list=[RuleReward(rl, None, actor)], train_iters=2, save_interval=0,
                             global_batch_size=4, n_samples_per_prompt=4, pad_token_id=0)
    hist = trainer.fit(SyntheticPromptLoader(4, 12, 63, seed=0, num_batches=100))
    assert len(hist) == 2
    for m in hist:
        assert m["train/num_gen_batches"] >= 1
        assert "actor/pg_loss" in m and m["actor/kl_loss"] == 0.0
        # every kept group has both hits and misses -> mean score strictly inside the reward range
        assert -1.0 < m["dapo/score/mean"] < 1.0
        assert m["timing/rollout"] > 0 and m["e2e_tps"] > 0


def test_ppo_with_critic_cpu():
    torch.manual_seed(0)
    actor, rl, gen = _configs("ray_ppo", adv_estimator="gae", use_kl_in_reward=True, kl_penalty="kl",
                              init_kl_coef=0.01, cliprange_value=0.5, critic_resource={"num_gpus": 1},
                              use_integrated_worker=True)
    critic_cfg = MegatronConfig(dict(model="tiny_qwen2", global_batch_size=4, micro_batch_size=4, seq_length=64,
                                     lr=1e-4, lr_decay_style="constant", stage="ray_ppo", train_iters=2, seed=1),
                                {"tiny_qwen2": {k: getattr(actor, k) for k in
                                                ("num_layers", "hidden_size", "ffn_hidden_size", "num_attention_heads",
                                                 "num_query_groups", "group_query_attention", "padded_vocab_size",
                                                 "add_qkv_bias", "normalization", "swiglu", "position_embedding_type",
                                                 "untie_embeddings_and_output_weights", "norm_epsilon", "rotary_base",
                                                 "max_position_embeddings")}})
    validate_rl_args(actor, actor, actor, rl, gen, critic_config=critic_cfg)
    worker = IntegratedWorker(actor, rl, gen, eos_token_id=63, pad_token_id=0, device="cpu")
    actor_group = SPMDWorkerGroup(worker, 1).initialize()
    critic_group = SPMDWorkerGroup(CriticWorker(critic_cfg, rl, gen, pad_token_id=0, device="cpu"), 1).initialize()
    trainer = RayPPOTrainer(actor_group, reward_list=[RuleReward(rl, None, actor)], critic_worker=critic_group,
                            train_iters=2, save_interval=0, global_batch_size=4, n_samples_per_prompt=4,
                            pad_token_id=0, use_kl_in_reward=True, kl_penalty="kl", init_kl_coef=0.01,
                            gamma=1.0, lam=0.95)
    before = critic_group.worker.model.module.rm_head.weight.detach().clone()
    hist = trainer.fit(iter(SyntheticPromptLoader(4, 12, 63, seed=0)))
    assert len(hist) == 2
    for m in hist:
        for k in ("critic/vf_loss", "critic/vf_clipfrac", "actor/pg_loss", "critic/values/mean",
                  "critic/returns/mean", "timing/update_critic", "timing/critic_model", "timing/kl"):
            assert k in m, k
    assert not torch.equal(before, critic_group.worker.model.module.rm_head.weight)


def test_grpo_lora_cpu():
    """LoRA GRPO: only adapters move, the backbone without adapters serves as the reference (no
    second model), the rollout engine runs on merged weights."""
    from test_e2e_grpo_cpu import build
    from mindspeed_rl_b200.trainer.grpo_trainer import RayGRPOTrainer

    torch.manual_seed(0)
    actor, rl, gen = build(n_prompts=4, n_samples=4, max_tokens=16, iters=2)
    actor.lora_r, actor.lora_alpha = 4, 8
    actor.lora_target_modules = ["linear_qkv", "linear_proj", "linear_fc1", "linear_fc2"]
    actor.lr = 1e-2
    worker = IntegratedWorker(actor, rl, gen, eos_token_id=1023, pad_token_id=0, device="cpu")
    group = SPMDWorkerGroup(worker, num_gpus=1).initialize()
    assert worker.ref_model is None and worker.reference is not None and worker.reference.disable_adapter
    core = worker.model.module
    before = {k: v.clone() for k, v in core.state_dict().items()}
    trainer = RayGRPOTrainer(group, reward_list=[RuleReward(rl, None, actor)], train_iters=2, save_interval=0,
                             adv_estimator="group_norm", kl_penalty="low_var_kl", init_kl_coef=0.001,
                             global_batch_size=4, n_samples_per_prompt=4, pad_token_id=0)
    hist = trainer.fit(iter(SyntheticPromptLoader(4, 32, 1024, seed=0)))
    assert len(hist) == 2 and "actor/kl_loss" in hist[0]
    after = core.state_dict()
    moved = [k for k in before if not torch.equal(before[k], after[k])]
    assert moved and all("lora_" in k for k in moved), moved
    assert sum(p.numel() for b in worker.model.buffers for p in b.params) == \
        sum(p.numel() for n, p in core.named_parameters() if "lora_" in n)


def test_grpo_partial_rollout_cpu():
    """Partial rollout: each round generates at most max_tokens / max_split new tokens; unfinished
    responses are continued (prompt + partial response) in a later round or iteration."""
    from test_e2e_grpo_cpu import build
    from mindspeed_rl_b200.trainer.grpo_trainer import RayGRPOTrainer

    torch.manual_seed(0)
    actor, rl, gen = build(n_prompts=4, n_samples=2, max_tokens=24, iters=2)
    rl.partial_rollout_max_split = 2
    worker = IntegratedWorker(actor, rl, gen, eos_token_id=1023, pad_token_id=0, device="cpu")
    group = SPMDWorkerGroup(worker, num_gpus=1).initialize()
    rounds = []
    inner = worker._generate_batch_partial

    def spy(batch, idx):
        rounds.append((batch["response_length"].reshape(-1).tolist(), batch["age"].reshape(-1).tolist()))
        return inner(batch, idx)

    worker._generate_batch_partial = spy
    trainer = RayGRPOTrainer(group, reward_list=[RuleReward(rl, None, actor)], train_iters=2, save_interval=0,
                             adv_estimator="group_norm", kl_penalty="low_var_kl", init_kl_coef=0.001,
                             global_batch_size=4, n_samples_per_prompt=2, pad_token_id=0,
                             partial_rollout_max_split=2)
    hist = trainer.fit(iter(SyntheticPromptLoader(4, 32, 1024, seed=0)))
    assert len(hist) == 2 and all(m["response_length/max"] <= 24 for m in hist)
    assert any(max(lens) == 0 for lens, _ in rounds), "no fresh prompts were generated"
    assert any(min(lens) == 12 for lens, _ in rounds), "no half-finished response was continued"


def test_grpo_multi_turn_tool_loop_cpu():
    """GRPO with the multi-turn tool loop inside the worker: every sample's first turn is followed by a tool
    turn (a scripted call to a registered tool), tool tokens are masked out of the loss (``response_mask``) and
    the number of tool calls is reported."""
    from test_e2e_grpo_cpu import build
    from test_tools_cpu import CharTokenizer, EchoTool  # noqa: F401  (registers the tool class)
    from mindspeed_rl_b200.tools.base import FunctionSchema, HermesToolParser, build_tool_map
    from mindspeed_rl_b200.trainer.grpo_trainer import RayGRPOTrainer

    torch.manual_seed(0)
    actor, rl, gen = build(n_prompts=2, n_samples=2, max_tokens=12, iters=1)
    rl.multi_turn_enable, rl.max_tool_calls, rl.max_parallel_calls = True, 1, 1
    rl.max_total_response_length, rl.max_tool_response_length, rl.tool_parser_format = 120, 16, "hermes"
    gen.max_model_len = 256
    gen.enable_prefix_caching = True
    worker = IntegratedWorker(actor, rl, gen, eos_token_id=-1, pad_token_id=0, device="cpu")
    group = SPMDWorkerGroup(worker, num_gpus=1).initialize()
    tok = CharTokenizer()
    worker.attach_tools(tok, build_tool_map([{"class_name": "EchoTool", "tool_schema": FunctionSchema("echo").to_openai()}]))

    class Scripted(HermesToolParser):
        def extract_tool_calls(self, ids):
            return self.extract_from_text('<tool_call>{"name": "echo", "arguments": {"k": 1}}</tool_call>')

    worker.multi_turn.parser = Scripted(tok)
    seen = {}
    inner = worker.actor.update

    def spy(batch, kl_ctrl=None):
        seen["mask"] = batch["response_mask"].clone()
        seen["len"] = batch["response_length"].reshape(-1).clone()
        return inner(batch, kl_ctrl)

    worker.actor.update = spy
    trainer = RayGRPOTrainer(group, reward_list=[RuleReward(rl, None, actor)], train_iters=1, save_interval=0,
                             adv_estimator="group_norm", kl_penalty="low_var_kl", init_kl_coef=0.001,
                             global_batch_size=2, n_samples_per_prompt=2, pad_token_id=0)
    hist = trainer.fit(iter(SyntheticPromptLoader(2, 16, 1024, seed=0)))
    assert len(hist) == 1 and hist[0]["tool_call_num/mean"] == 1.0
    assert hist[0]["tool_call_num/max"] == 1 and hist[0]["response_length/max"] <= 120
    assert hist[0]["response_length/min"] > 12                                                # a tool turn was added
    mask, lens = seen["mask"], seen["len"]
    for row, n in zip(mask, lens.tolist()):
        live = row[:n]
        assert int(live.sum()) < n and int(live[:12].sum()) == 12 and int(live[12]) == 0   # first turn counts, tool turn does not


def test_dapo_dynamic_sampling_with_partial_rollout_cpu():
    """Dynamic sampling and partial rollout together (the combination of the DAPO benchmark configuration): the
    rollout writes rounds of at most max_tokens / 2 new tokens into the sampling store, finished groups are
    judged and the informative ones moved to the training store, unfinished ones continue beside the next
    batch of prompts.  The samples of one prompt must differ although the sampling seed is fixed."""
    torch.manual_seed(0)
    actor, rl, gen = _configs("ray_dapo", clip_higher_enable=True, clip_ratio_low=0.2, clip_ratio_high=0.28,
                              filter_groups_enable=True, filter_groups_metric="contains_token_7",
                              filter_groups_max_batches=20, filter_groups_train_batch_size=2, token_level_loss=True,
                              partial_rollout_max_split=2)
    validate_rl_args(actor, None, actor, rl, gen)
    worker = IntegratedWorker(actor, rl, gen, eos_token_id=63, pad_token_id=0, device="cpu", with_reference=False)
    group = SPMDWorkerGroup(worker, 1).initialize()
    trainer = RayDAPOTrainer(group, reward_list=[RuleReward(rl, None, actor)], train_iters=2, save_interval=0,
                             global_batch_size=4, n_samples_per_prompt=4, pad_token_id=0,
                             partial_rollout_max_split=2)
    store = trainer.sampling_transfer_dock
    assert store.enable_partial_rollout and store.max_len == 2 * 4 * 4 and not trainer.transfer_dock.enable_partial_rollout
    groups_seen = []
    judge = trainer.dynamic_sampling

    def spy():
        rows = [r.tolist() for r in store.experience_data["responses"][:16] if r is not None]
        groups_seen.extend(rows[i:i + 4] for i in range(0, len(rows) - 3, 4))
        return judge()

    trainer.dynamic_sampling = spy
    hist = trainer.fit(SyntheticPromptLoader(4, 12, 63, seed=0, num_batches=200))
    assert len(hist) == 2 and all(m["train/num_gen_batches"] >= 1 and "actor/pg_loss" in m for m in hist)
    assert all(-1.0 < m["dapo/score/mean"] < 1.0 and m["response_length/max"] <= 16 for m in hist)
    assert groups_seen and all(len({tuple(r) for r in g}) > 1 for g in groups_seen), "identical samples in a group"
