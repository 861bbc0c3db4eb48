"""Every shipped recipe parses, passes cross-config validation and derives its dispatch sizes;
unknown keys are rejected; the catalogue of model architectures loads."""
import glob
import os

import pytest

from mindspeed_rl_b200.config import MegatronConfig, RLConfig, compose, parse_training_config
from mindspeed_rl_b200.config.loader import load_model_catalogue

ROOT = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "configs")
RECIPES = sorted(os.path.splitext(os.path.basename(p))[0] for p in glob.glob(os.path.join(ROOT, "*.yaml")))


@pytest.mark.parametrize("name", [r for r in RECIPES if not r.startswith("dpo_")])
def test_recipe_validates(name):
    cfg = compose(name)
    out = parse_training_config(cfg, with_critic=name.startswith("ppo_"))
    actor, rl, gen = out["actor_config"], out["rl_config"], out["generate_config"]
    gpus = rl.actor_resource["num_npus"]
    mp = actor.tensor_model_parallel_size * actor.pipeline_model_parallel_size * (actor.context_parallel_size or 1)
    assert gpus % mp == 0 and gpus % gen.infer_tensor_parallel_size == 0
    assert rl.actor_rollout_dispatch_size and rl.actor_rollout_dispatch_size > 0
    assert rl.mini_batch_size % rl.n_samples_per_prompt == 0          # scaled by n during validation
    assert actor.pad_to_multiple_of == actor.tensor_model_parallel_size * (actor.context_parallel_size or 1)
    if name.startswith("ppo_"):
        assert out["critic_config"] is not None and rl.critic_resource is not None
    # the pipeline stages hold every layer exactly once (uneven stage sizes come from num_layer_list)
    from mindspeed_rl_b200.reshard.planner import pipeline_layout
    stages = pipeline_layout(actor, actor.pipeline_model_parallel_size)
    layers = sorted(l for st in stages for chunk in st for l in chunk)
    assert len(stages) == actor.pipeline_model_parallel_size and layers == list(range(len(layers)))
    assert len(layers) == actor.num_layers - len(actor.noop_layers or [])


def test_dpo_recipe_and_model_catalogue():
    cfg = compose("dpo_qwen3_30b_a3b_b200")
    mt = MegatronConfig(cfg["megatron_training"], cfg["model"])
    assert mt.stage == "dpo" and mt.is_pairwise_dataset and mt.num_experts == 128
    cat = load_model_catalogue(["qwen25_7b", "qwen3_8b", "deepseekv3_671b"])
    assert cat["qwen25_7b"]["num_layers"] == 28 and cat["qwen3_8b"]["qk_layernorm"]
    assert cat["deepseekv3_671b"]["multi_latent_attention"]


def test_unknown_keys_are_rejected():
    with pytest.raises(ValueError):
        RLConfig({"no_such_option": 1})
    with pytest.raises(ValueError):
        MegatronConfig({"model": "tiny_qwen2", "definitely_not_a_knob": True}, compose("grpo_tiny_cpu")["model"])


def test_dataset_and_tool_configs_load():
    import yaml

    from mindspeed_rl_b200.tools.base import build_tool_map
    for p in glob.glob(os.path.join(ROOT, "datasets", "*.yaml")):
        d = yaml.safe_load(open(p))
        assert {"input", "output_prefix", "handler_name", "tokenizer_name_or_path"} <= set(d)
    for p in glob.glob(os.path.join(ROOT, "tools", "*.yaml")):
        tools = build_tool_map(yaml.safe_load(open(p))["tools"])
        assert len(tools) == 1


def test_tied_embeddings_with_pipeline_parallel_are_refused():
    """The first and the last pipeline stage would each train a copy of the tied matrix and nothing
    keeps the copies equal, so the validator stops such a run."""
    cfg = compose("grpo_tiny_cpu", None, ["actor_config.pipeline_model_parallel_size=2",
                                          "rl_config.actor_resource.num_gpus=2",
                                          "+model.tiny_qwen2.untie_embeddings_and_output_weights=false"])
    with pytest.raises(ValueError, match="tied input/output embeddings"):
        parse_training_config(cfg)


def test_layer_lists_are_read_from_comma_separated_text():
    from mindspeed_rl_b200.config.training_config import MegatronConfig
    from mindspeed_rl_b200.reshard.planner import stage_layers
    c = MegatronConfig({"num_layers": 64, "pipeline_model_parallel_size": 4, "num_layer_list": "16,17,16,15",
                        "noop_layers": "0, 63"})
    assert c.num_layer_list == [16, 17, 16, 15] and c.noop_layers == [0, 63]
    assert [len(s) for s in stage_layers(64, 4, c.num_layer_list)] == [16, 17, 16, 15]
    assert MegatronConfig({"num_layers": 4}).num_layer_list is None
    with pytest.raises(ValueError):
        MegatronConfig({"num_layers": 4, "num_layer_list": "2,x"})


def test_vision_language_model_file_sets_the_stage_layout(tmp_path):
    import json
    from mindspeed_rl_b200.config.training_config import MegatronConfig
    path = tmp_path / "model.json"
    path.write_text(json.dumps({"image_encoder": {"vision_encoder": {"pipeline_num_layers": [32, 0]}},
                                "text_decoder": {"pipeline_num_layers": [12, 16]}}))
    c = MegatronConfig({"num_layers": 28})
    c.update({"model": "qwen25vl"}, str(path))
    c._finalize()
    assert c.num_layer_list == [[32, 0], [12, 16]] and c.mm_model == str(path)
    path.write_text(json.dumps({"text_decoder": {}}))
    with pytest.raises(ValueError):
        MegatronConfig({"num_layers": 28}).update({"model": "x"}, str(path))
    with pytest.raises(FileNotFoundError):
        MegatronConfig({"num_layers": 28}).update({"model": "x"}, str(tmp_path / "missing.json"))


def test_layouts_that_do_not_divide_are_refused():
    from mindspeed_rl_b200.config.loader import apply_overrides
    base = compose("dapo_qwen3_30b_a3b_b200")
    parse_training_config(base)                                             # the shipped recipe is fine
    for bad in (["actor_config.moe_tp_extend_ep=false"],                     # experts would be cut by TP
                ["megatron_training.sequence_parallel=false"],               # every TP rank would route every token
                ["generate_config.infer_expert_parallel_size=48"],           # 128 experts over 48 ranks
                ["actor_config.tensor_model_parallel_size=8", "rl_config.actor_resource.num_gpus=16"]):   # 4 KV heads over TP8
        with pytest.raises(ValueError):
            parse_training_config(apply_overrides(compose("dapo_qwen3_30b_a3b_b200"), bad))
    with pytest.raises(ValueError):                                          # 28 heads over TP8
        parse_training_config(apply_overrides(compose("grpo_qwen25_7b_b200"),
                                              ["actor_config.tensor_model_parallel_size=8"]))


def test_partial_rollout_combinations_that_are_not_served_are_refused():
    from mindspeed_rl_b200.config.loader import apply_overrides
    ok = apply_overrides(compose("grpo_tiny_cpu"), ["rl_config.partial_rollout_max_split=2"])
    assert parse_training_config(ok)["rl_config"].partial_rollout_max_split == 2
    for bad in (["rl_config.guarantee_order=true"],
                ["rl_config.multi_turn_enable=true", "rl_config.async_engine=true",
                 "rl_config.max_total_response_length=128"]):
        with pytest.raises(ValueError):
            parse_training_config(apply_overrides(compose("grpo_tiny_cpu"),
                                                  ["rl_config.partial_rollout_max_split=2"] + bad))


def test_example_scripts_point_at_existing_entry_points_and_recipes():
    """Every launch script names a command-line entry point and a recipe that exist, and the recipe's algorithm
    matches the entry point; the scripts parse as shell."""
    import re
    import subprocess
    repo = os.path.dirname(ROOT)
    scripts = sorted(glob.glob(os.path.join(repo, "examples", "*", "*.sh")))
    assert len(scripts) >= 20
    stages = {"train_grpo.py": "ray_grpo", "train_dapo.py": "ray_dapo", "train_ppo.py": "ray_ppo", "train_dpo.py": "dpo"}
    launched = 0
    for path in scripts + [os.path.join(repo, "examples", "common.sh")]:
        assert subprocess.run(["bash", "-n", path]).returncode == 0, path
        text = open(path).read()
        for cli in re.findall(r"cli/([a-z_]+\.py)", text):
            assert os.path.isfile(os.path.join(repo, "cli", cli)), (path, cli)
        m = re.search(r"^launch_trainer (\S+) (\S+)", text, re.MULTILINE)
        if m:
            launched += 1
            cli, recipe = m.groups()
            assert os.path.isfile(os.path.join(repo, "cli", cli)), (path, cli)
            assert os.path.isfile(os.path.join(ROOT, recipe + ".yaml")), (path, recipe)
            assert compose(recipe)["megatron_training"]["stage"] == stages[cli], (path, recipe)
    assert launched >= 19
    # every shipped full-size recipe has a launch script
    named = {re.search(r"^launch_trainer \S+ (\S+)", open(p).read(), re.MULTILINE) for p in scripts}
    named = {m.group(1) for m in named if m}
    assert {r for r in RECIPES if r.endswith("_b200")} <= named, sorted({r for r in RECIPES if r.endswith("_b200")} - named)
