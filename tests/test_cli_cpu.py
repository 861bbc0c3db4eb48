"""Command-line entry points end to end on CPU with the whitespace-integer tokenizer: raw JSON lines ->
``cli/preprocess_data.py`` -> packed ``.bin/.idx`` -> datasets / the DPO trainer."""
import importlib
import json
import os
import random
import sys

import numpy as np
import pytest
import yaml

ROOT = os.path.join(os.path.dirname(__file__), "..")


def _cli(name):
    if os.path.abspath(ROOT) not in [os.path.abspath(p) for p in sys.path]:
        sys.path.insert(0, os.path.abspath(ROOT))
    return importlib.import_module(f"cli.{name}")        # importable by name: its workers are pickled by reference


def _numbers(rng, n):
    return " ".join(str(rng.randint(3, 90)) for _ in range(n))


def test_preprocess_pairwise_then_dpo_cli(tmp_path):
    rng = random.Random(0)
    rows = [{"question": _numbers(rng, 6), "chosen": _numbers(rng, 4), "rejected": _numbers(rng, 5), "system": ""}
            for _ in range(16)]
    (tmp_path / "pairs.jsonl").write_text("\n".join(json.dumps(r) for r in rows) + "\n")
    (tmp_path / "out").mkdir()
    yaml.safe_dump(dict(input=str(tmp_path / "pairs.jsonl"), tokenizer_name_or_path="none", tokenizer_type="Identity",
                        pad_vocab_size_to=96, output_prefix=str(tmp_path / "out" / "pairs"),
                        handler_name="AlpacaStylePairwiseHandler", workers=1, prompt_type="empty",
                        map_keys={"prompt": "question", "query": "", "system": "system"}),
                   open(tmp_path / "pairs.yaml", "w"))
    prefixes = _cli("preprocess_data").main(["pairs", "--config-dir", str(tmp_path)])
    assert set(prefixes) == {"chosen_input_ids", "chosen_labels", "rejected_input_ids", "rejected_labels"}
    for p in prefixes.values():
        assert os.path.getsize(p + ".bin") > 0 and os.path.getsize(p + ".idx") > 0

    # the first pair comes back as written: prompt tokens masked in the labels, answers kept
    from mindspeed_rl_b200.datasets.indexed_dataset import get_packed_indexed_dataset
    ds = get_packed_indexed_dataset(str(tmp_path / "out" / "pairs"), None, True)
    first = ds[0]
    q = [int(t) for t in rows[0]["question"].split()]
    c = [int(t) for t in rows[0]["chosen"].split()]
    ids, labels = list(first["chosen_input_ids"]), list(first["chosen_labels"])
    assert ids[:len(q)] == q and ids[len(q):len(q) + len(c)] == c
    assert all(l == -100 for l in labels[:len(q)]) and labels[len(q):len(q) + len(c)] == c

    recipe = {"defaults": [{"model": ["tiny_qwen2"]}],
              "megatron_training": dict(model="tiny_qwen2", stage="dpo", is_pairwise_dataset=True, dpo_beta=0.1,
                                        dpo_loss_type="sigmoid", tensor_model_parallel_size=1,
                                        pipeline_model_parallel_size=1, global_batch_size=4, micro_batch_size=1,
                                        seq_length=64, train_iters=3, lr=1e-4, min_lr=0, lr_decay_style="constant",
                                        weight_decay=0.0, clip_grad=1.0, bf16=False, tokenizer_type="Identity",
                                        tokenizer_name_or_path="none", data_path=str(tmp_path / "out" / "pairs"),
                                        split="100,0,0", seed=1234, distributed_backend="gloo", log_interval=1,
                                        save=str(tmp_path / "ckpt"), save_interval=3)}
    yaml.safe_dump(recipe, open(tmp_path / "dpo_tiny.yaml", "w"))
    hist = _cli("train_dpo").main(["--config-name", "dpo_tiny", "--config-dir", str(tmp_path)])
    assert len(hist) == 3
    assert abs(hist[0]["dpo/loss"] - float(np.log(2.0))) < 1e-5          # policy == reference at the start
    assert all(np.isfinite(h["dpo/loss"]) and h["grad_norm"] > 0 and h["samples_per_sec"] > 0 for h in hist)
    assert (tmp_path / "ckpt" / "latest_checkpointed_iteration.txt").read_text().strip() == "3"


def test_preprocess_prompts_in_parts_and_read_back(tmp_path):
    """RL prompts with reference answers, tokenised by two worker processes and merged; the prompt dataset
    serves every row once per epoch and keeps its shuffle index on disk."""
    rng = random.Random(1)
    rows = [{"problem": _numbers(rng, 5 + i % 3), "answer": str(i)} for i in range(20)]
    (tmp_path / "prompts.jsonl").write_text("\n".join(json.dumps(r) for r in rows) + "\n")
    (tmp_path / "out").mkdir()
    yaml.safe_dump(dict(input=str(tmp_path / "prompts.jsonl"), tokenizer_name_or_path="none", tokenizer_type="Identity",
                        pad_vocab_size_to=96, output_prefix=str(tmp_path / "out" / "data"),
                        handler_name="R1AlpacaStyleInstructionHandler", workers=2, n_subs=2, prompt_type="empty",
                        dataset_additional_keys=["labels"],
                        map_keys={"prompt": "problem", "query": "", "response": "answer", "system": ""}),
                   open(tmp_path / "prompts.yaml", "w"))
    prefixes = _cli("preprocess_data").main(["prompts", "--config-dir", str(tmp_path)])
    assert {"input_ids", "labels"} <= set(prefixes)

    from mindspeed_rl_b200.datasets.prompt_dataset import PromptDataset, build_train_valid_test_datasets
    extra = type("A", (), dict(is_pairwise_dataset=False, dataset_additional_keys=["labels"], max_prompt_length=None))()
    train, valid, _ = build_train_valid_test_datasets(str(tmp_path / "out" / "data"), "100,0,0", 64, [20, 0, 0],
                                                      PromptDataset, None, seed=3, extra_param=extra)
    assert valid is None and len(train) == 20
    seen = sorted(tuple(int(t) for t in train[i]["input_ids"]) for i in range(20))
    want = sorted(tuple(int(t) for t in r["problem"].split()) for r in rows)
    assert seen == want
    answers = sorted(int(train[i]["labels"][0]) for i in range(20))
    assert answers == list(range(20))
    assert any(f.endswith(".npy") for f in os.listdir(tmp_path / "out")), "no shuffle-index cache was written"


def test_convert_ckpt_cli_round_trip(tmp_path):
    """HF layout -> mcore shards for TP2 x PP2 -> HF layout through the command line, for the tiny architecture;
    the mcore shards also load into a TP1 model built from the same architecture file."""
    import torch
    from mindspeed_rl_b200.checkpoint import convert as C
    from mindspeed_rl_b200.config import MegatronConfig
    from mindspeed_rl_b200.config.loader import load_model_catalogue
    from mindspeed_rl_b200.models.gpt import GPTModel
    from mindspeed_rl_b200.models.transformer_config import TransformerConfig

    cfg = MegatronConfig({"model": "tiny_qwen2"}, load_model_catalogue(["tiny_qwen2"]))
    model = GPTModel(TransformerConfig.from_megatron(cfg, params_dtype=torch.float32), device="cpu", seed=2)
    hf = C.mcore_to_hf({(0, 0, 0): model.state_dict()}, cfg)
    C.save_hf_state(hf, str(tmp_path / "hf"))
    cli = _cli("convert_ckpt")
    cli.main(["hf2mcore", "--model", "tiny_qwen2", "--load", str(tmp_path / "hf"), "--save", str(tmp_path / "mcore"),
              "--tp", "2", "--pp", "2"])
    assert (tmp_path / "mcore" / "latest_checkpointed_iteration.txt").exists()
    cli.main(["mcore2hf", "--model", "tiny_qwen2", "--load", str(tmp_path / "mcore"), "--save", str(tmp_path / "hf2"),
              "--tp", "2", "--pp", "2"])
    back = C.load_hf_state(str(tmp_path / "hf2"))
    assert set(back) == set(hf)
    for k in hf:
        assert torch.equal(back[k], hf[k]), k
    cli.main(["hf2mcore", "--model", "tiny_qwen2", "--load", str(tmp_path / "hf2"), "--save", str(tmp_path / "one")])
    again = GPTModel(TransformerConfig.from_megatron(cfg, params_dtype=torch.float32), device="cpu", seed=5)
    missing, unexpected = again.load_state_dict(C.read_mcore(str(tmp_path / "one"), 1, 1)[(0, 0, 0)], strict=False)
    assert not missing and not unexpected
    for (n, a), (_, b) in zip(model.named_parameters(), again.named_parameters()):
        assert torch.equal(a, b), n


def test_eplb_map_cli_from_dumped_counts(tmp_path):
    """Routing counts dumped by two rollout ranks -> placement map with one redundant slot per device: every
    expert is hosted somewhere, the hottest expert twice, and the slots of a layer fill all devices evenly."""
    layers, experts, gpus = 3, 8, 4
    rng = random.Random(4)
    for rank in range(2):
        data = {str(l): {str(e): rng.randint(1, 50) + (400 if e == 5 else 0) for e in range(experts)}
                for l in range(layers)}
        (tmp_path / f"eplb_token_collects_{rank}.json").write_text(json.dumps(data))
    out = tmp_path / "expert_map.json"
    _cli("eplb_generate_map").main(["--json_folder", str(tmp_path), "--num_gpus", str(gpus), "--num_redundancy", "1",
                                    "--output", str(out)])
    emap = json.loads(out.read_text())
    assert emap["moe_layer_count"] == layers
    for layer in emap["layer_list"]:
        hosted = [d["device_expert"] for d in layer["device_list"]]
        assert len(hosted) == gpus and all(len(h) == experts // gpus + 1 for h in hosted)
        flat = [e for h in hosted for e in h]
        assert set(flat) == set(range(experts)) and flat.count(5) >= 2
        assert all(len(set(h)) == len(h) for h in hosted)


def test_grpo_saves_and_resumes(tmp_path):
    """Two iterations with a checkpoint after each; a second run that loads the checkpoint starts at iteration 2,
    has the same weights, skips the prompts already used and trains one more iteration."""
    import torch
    from mindspeed_rl_b200.checkpoint.mcore import load_args_from_checkpoint
    from mindspeed_rl_b200.config import compose
    from mindspeed_rl_b200.config.loader import apply_overrides
    from mindspeed_rl_b200.runtime.launch import run_rl

    save = str(tmp_path / "ckpt")
    base = ["megatron_training.global_batch_size=4", "rl_config.mini_batch_size=4", "rl_config.n_samples_per_prompt=2",
            "generate_config.sampling_config.max_tokens=8", "megatron_training.seq_length=96",
            f"actor_config.save={save}", "megatron_training.save_interval=1", "actor_config.lr=1e-3"]
    hist = run_rl(apply_overrides(compose("grpo_tiny_cpu"), base + ["megatron_training.train_iters=2"]), "grpo")
    assert len(hist) == 2
    assert (tmp_path / "ckpt" / "latest_checkpointed_iteration.txt").read_text().strip() == "2"
    assert (tmp_path / "ckpt" / "iter_0000001").is_dir() and (tmp_path / "ckpt" / "iter_0000002").is_dir()
    args = load_args_from_checkpoint(save)
    assert args is not None and int(getattr(args, "num_layers", args.get("num_layers") if isinstance(args, dict) else 0)) == 2
    state = torch.load(tmp_path / "ckpt" / "iter_0000002" / "mp_rank_00" / "model_optim_rng.pt", weights_only=False)
    assert state["iteration"] == 2 and "optimizer" in state and "opt_param_scheduler" in state
    resumed = run_rl(apply_overrides(compose("grpo_tiny_cpu"),
                                     base + ["megatron_training.train_iters=3", f"actor_config.load={save}"]), "grpo")
    assert len(resumed) == 1                                   # iterations 1 and 2 are not repeated
    assert (tmp_path / "ckpt" / "latest_checkpointed_iteration.txt").read_text().strip() == "3"


def test_expert_load_collection_to_placement_map_to_rollout(tmp_path):
    """The load-balancing workflow end to end on one rank: a run of a small expert model records how many tokens
    every expert received during rollout, the map generator turns the records into a placement with a redundant
    slot, and a second run rolls out with that placement."""
    from mindspeed_rl_b200.config import compose
    from mindspeed_rl_b200.runtime.launch import run_rl

    moe = ["+model.tiny_qwen2.num_experts=4", "+model.tiny_qwen2.moe_router_topk=2",
           "+model.tiny_qwen2.moe_ffn_hidden_size=32", "+model.tiny_qwen2.norm_topk_prob=true",
           "megatron_training.global_batch_size=4", "rl_config.mini_batch_size=4", "rl_config.n_samples_per_prompt=2",
           "generate_config.sampling_config.max_tokens=8", "megatron_training.train_iters=1"]
    stats = tmp_path / "load"
    hist = run_rl(compose("grpo_tiny_cpu", None, moe + ["generate_config.eplb_token_collects=true",
                                                        f"generate_config.eplb_token_save_path={stats}"]), "grpo")
    assert len(hist) == 1
    record = json.loads((stats / "eplb_token_collects_0.json").read_text())
    assert sorted(record, key=int) == ["0", "1"]                     # both layers are expert layers
    for layer in record.values():
        assert sorted(layer, key=int) == ["0", "1", "2", "3"] and sum(layer.values()) > 0
    # prompts 4 x 2 samples, prefill + 8 decode steps, top-2 routing: every token is counted twice per layer
    assert sum(record["0"].values()) == sum(record["1"].values()) and sum(record["0"].values()) % 2 == 0
    out = tmp_path / "expert_map.json"
    _cli("eplb_generate_map").main(["--json_folder", str(stats), "--num_gpus", "2", "--num_redundancy", "1",
                                    "--output", str(out)])
    emap = json.loads(out.read_text())
    for li, layer in enumerate(emap["layer_list"]):
        hosted = [d["device_expert"] for d in layer["device_list"]]
        assert [len(h) for h in hosted] == [3, 3] and set(hosted[0]) | set(hosted[1]) == {0, 1, 2, 3}
        assert all(len(set(h)) == 3 for h in hosted)                    # no expert twice on one device
    # one device cannot host five slots of four experts without a duplicate: refused with a clear message
    with pytest.raises(ValueError, match="same expert twice"):
        _cli("eplb_generate_map").main(["--json_folder", str(stats), "--num_gpus", "1", "--num_redundancy", "1",
                                        "--output", str(out)])


def test_vision_language_run_through_the_launcher(tmp_path):
    """JSON-lines rows with inline images -> multimodal dataset -> vision stage (architecture from the recipe's
    ``vit_config`` section) -> rollout, reference and update of one GRPO iteration."""
    from mindspeed_rl_b200.config import compose
    from mindspeed_rl_b200.runtime.launch import run_rl

    rng = np.random.default_rng(0)
    with open(tmp_path / "rows.jsonl", "w") as f:
        for i in range(8):
            img = (rng.random((28, 42, 3)) * 255).astype(np.uint8).tolist()
            f.write(json.dumps({"prompt": f"5 6 <image> 7 {8 + i}", "images": [img], "answer": str(i)}) + "\n")
    cfg = compose("grpo_tiny_cpu", None, [
        "megatron_training.global_batch_size=4", "rl_config.mini_batch_size=4", "rl_config.n_samples_per_prompt=2",
        "generate_config.sampling_config.max_tokens=8", "megatron_training.train_iters=1",
        f"megatron_training.data_path={tmp_path / 'rows.jsonl'}", "+rl_config.is_multimodal=true",
        "+rl_config.reuse_image_embeds=true", "generate_config.enable_prefix_caching=false",
        "rl_config.use_remove_padding=false", "+megatron_training.image_token_id=1000",
        "+megatron_training.vision_start_token_id=1001", "+megatron_training.vision_end_token_id=1002",
        "+vit_config.hidden_size=32", "+vit_config.num_layers=1", "+vit_config.num_attention_heads=2",
        "+vit_config.ffn_hidden_size=48", "+rl_config.max_prompt_length=96"])
    hist = run_rl(cfg, "grpo")
    assert len(hist) == 1 and hist[0]["timing/vit_image_emb"] > 0 and hist[0]["timing/rollout"] > 0
    # 4 text tokens + start marker + 3 image placeholders (2 x 3 patches merged 2 x 2 -> ... ) + end marker
    assert hist[0]["prompt_length/mean"] == hist[0]["prompt_length/max"] > 6


def test_ppo_and_dapo_through_the_launcher():
    """One iteration each of PPO (critic group built from the recipe's critic section) and DAPO (no reference
    model) through the launcher that the command-line entry points call."""
    from mindspeed_rl_b200.config import compose
    from mindspeed_rl_b200.runtime.launch import run_rl
    small = ["megatron_training.global_batch_size=4", "rl_config.mini_batch_size=4", "rl_config.n_samples_per_prompt=2",
             "generate_config.sampling_config.max_tokens=8", "megatron_training.train_iters=1"]
    h = run_rl(compose("grpo_tiny_cpu", None, small + [
        "megatron_training.stage=ray_ppo", "rl_config.adv_estimator=gae", "+critic_config.model=tiny_qwen2",
        "+critic_config.micro_batch_size=4", "+critic_config.lr=1e-5", "+rl_config.critic_resource.num_gpus=1"]), "ppo")
    assert len(h) == 1 and "critic/vf_loss" in h[0] and "critic/values/mean" in h[0] and h[0]["timing/update_critic"] > 0
    # the same with every training-state offload switched on: the critic parks its state between its stages
    h = run_rl(compose("grpo_tiny_cpu", None, small + [
        "megatron_training.stage=ray_ppo", "rl_config.adv_estimator=gae", "+critic_config.model=tiny_qwen2",
        "+critic_config.micro_batch_size=4", "+critic_config.lr=1e-5", "+rl_config.critic_resource.num_gpus=1",
        "megatron_training.train_iters=2", "+generate_config.offload_train_param=true",
        "+generate_config.offload_train_grad=true", "+generate_config.offload_train_optimizer=true"]), "ppo")
    assert len(h) == 2 and all(m["critic/vf_loss"] >= 0 and m["actor/grad_norm"] >= 0 for m in h)

    h = run_rl(compose("grpo_tiny_cpu", None, small + [
        "megatron_training.stage=ray_dapo", "+rl_config.clip_higher_enable=true", "+rl_config.clip_ratio_low=0.2",
        "+rl_config.clip_ratio_high=0.28", "+rl_config.token_level_loss=true", "rl_config.init_kl_coef=0.0"]), "dapo")
    assert len(h) == 1 and "dapo/score/mean" in h[0] and h[0]["actor/kl_loss"] == 0.0
    assert "timing/reference_model" not in h[0] or h[0]["timing/reference_model"] == 0


def test_profiler_trace_and_key_data_dump_through_the_launcher(tmp_path):
    """A run with the profiler on for the update stage and the accuracy-debugging dump on for the first iteration
    leaves a trace file, the configurations and per-stage statistics of prompts, responses, log-probs, advantages
    and losses (what the reference's system test checks after its PPO run)."""
    from mindspeed_rl_b200.config import compose
    from mindspeed_rl_b200.runtime.launch import run_rl
    prof, dump = tmp_path / "prof", tmp_path / "dump"
    cfg = compose("grpo_tiny_cpu", None, [
        "megatron_training.global_batch_size=4", "rl_config.mini_batch_size=4", "rl_config.n_samples_per_prompt=2",
        "generate_config.sampling_config.max_tokens=8", "megatron_training.train_iters=2",
        "+profiler_config.integrated.profile=true", "+profiler_config.integrated.stage=actor_update",
        f"+profiler_config.integrated.profile_save_path={prof}", "+profiler_config.integrated.profile_step_start=1",
        "+profiler_config.integrated.profile_step_end=2", "+msprobe_config.msprobe=true",
        f"+msprobe_config.dump_path={dump}", "+msprobe_config.key_data_dump=true",
        "+msprobe_config.configurations_dump=true", "+msprobe_config.step_start=0", "+msprobe_config.step_end=0"])
    assert len(run_rl(cfg, "grpo")) == 2
    traces = [f for _, _, fs in os.walk(prof) for f in fs]
    assert traces and any(f.endswith(".json") for f in traces)
    assert (dump / "configurations.json").exists()
    step0 = dump / "step0" / "rank0"
    # one mini-batch per iteration: the old log-probs equal the current ones and that stage is skipped
    assert sorted(p.name for p in step0.iterdir()) == ["actor_generate.json", "actor_update.json", "ref_log_prob.json"]
    upd = json.loads((step0 / "actor_update.json").read_text())
    assert {"responses", "advantages", "ref_log_prob", "actor/pg_loss", "actor/grad_norm"} <= set(upd)
    assert upd["ref_log_prob"]["nan"] == 0 and upd["ref_log_prob"]["max"] <= 0.0
    ref = json.loads((step0 / "ref_log_prob.json").read_text())
    assert ref["ref_log_prob"]["numel"] > 0 and ref["ref_log_prob"]["inf"] == 0
    gen = json.loads((step0 / "actor_generate.json").read_text())
    assert gen["responses"]["numel"] == 4 * 2 * 8 and gen["prompt_length"]["mean"] == 64.0
    assert not (dump / "step1").exists()                              # outside the requested step range


def test_critic_statistics_in_the_dump(tmp_path):
    from mindspeed_rl_b200.config import compose
    from mindspeed_rl_b200.runtime.launch import run_rl
    dump = tmp_path / "dump"
    h = run_rl(compose("grpo_tiny_cpu", None, [
        "megatron_training.global_batch_size=4", "rl_config.mini_batch_size=4", "rl_config.n_samples_per_prompt=2",
        "generate_config.sampling_config.max_tokens=8", "megatron_training.train_iters=1",
        "megatron_training.stage=ray_ppo", "rl_config.adv_estimator=gae", "+critic_config.model=tiny_qwen2",
        "+critic_config.micro_batch_size=4", "+critic_config.lr=1e-5", "+rl_config.critic_resource.num_gpus=1",
        "+msprobe_config.msprobe=true", f"+msprobe_config.dump_path={dump}", "+msprobe_config.key_data_dump=true",
        "+msprobe_config.critic_train_dump=true", "+msprobe_config.step_start=0", "+msprobe_config.step_end=0"]), "ppo")
    assert len(h) == 1
    files = sorted(p.name for p in (dump / "step0" / "rank0").iterdir())
    assert files == ["critic_update.json"]                      # only the chosen stage is recorded
    rec = json.loads((dump / "step0" / "rank0" / "critic_update.json").read_text())
    assert {"values", "returns", "critic/vf_loss"} <= set(rec) and rec["values"]["nan"] == 0


def test_ppo_resumes_actor_and_critic(tmp_path):
    """PPO writes a checkpoint per trainable role; a second run resumes both: one more iteration is trained and the
    critic's optimizer carries on from its saved step count."""
    import torch
    from mindspeed_rl_b200.config import compose
    from mindspeed_rl_b200.runtime.launch import run_rl
    actor_dir, critic_dir = tmp_path / "actor", tmp_path / "critic"
    base = ["megatron_training.global_batch_size=4", "rl_config.mini_batch_size=4", "rl_config.n_samples_per_prompt=2",
            "generate_config.sampling_config.max_tokens=8", "megatron_training.stage=ray_ppo",
            "rl_config.adv_estimator=gae", "+critic_config.model=tiny_qwen2", "+critic_config.micro_batch_size=4",
            "+critic_config.lr=1e-3", "+rl_config.critic_resource.num_gpus=1", f"actor_config.save={actor_dir}",
            f"+critic_config.save={critic_dir}", "megatron_training.save_interval=1"]
    assert len(run_rl(compose("grpo_tiny_cpu", None, base + ["megatron_training.train_iters=2"]), "ppo")) == 2
    resumed = run_rl(compose("grpo_tiny_cpu", None, base + [
        "megatron_training.train_iters=3", f"actor_config.load={actor_dir}", f"+critic_config.load={critic_dir}"]), "ppo")
    assert len(resumed) == 1
    for d in (actor_dir, critic_dir):
        assert (d / "latest_checkpointed_iteration.txt").read_text().strip() == "3"
    state = torch.load(critic_dir / "iter_0000003" / "mp_rank_00" / "model_optim_rng.pt", weights_only=False)
    optim = torch.load(critic_dir / "iter_0000003" / "mp_rank_00" / "distrib_optim.pt", weights_only=False)
    assert state["iteration"] == 3 and optim["step"] == 3
    assert any(k.startswith("rm_head") for k in state["model"])
