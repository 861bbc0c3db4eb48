"""Weight-name adaptors, optimizer config, rollout-engine contract."""
import pytest
import torch

from mindspeed_rl_b200.optim.optimizer_config import OptimizerConfig
from mindspeed_rl_b200.reshard.weight_adaptor import get_weight_adaptor
from mindspeed_rl_b200.rollout.base_engine import BaseInferEngine
from mindspeed_rl_b200.rollout.engine import LLMEngine


def test_weight_adaptor_names_round_trip_and_pipeline_split():
    ad = get_weight_adaptor("Qwen3MoeForCausalLM")
    t = ad.replace_name_i2t("model.layers.17.self_attn.qkv_proj.weight")
    assert t == "decoder.layers.17.self_attention.linear_qkv.weight"
    assert ad.replace_name_t2i(t) == "model.layers.17.self_attn.qkv_proj.weight"
    assert ad.replace_name_i2t("model.layers.3.mlp.experts.w13_weight") == "decoder.layers.3.mlp.experts.weight1"
    assert ad.replace_name_i2t("model.layers.3.self_attn.q_norm.weight").endswith("q_layernorm.weight")
    with pytest.raises(KeyError):
        get_weight_adaptor("Qwen2ForCausalLM").replace_name_i2t("model.layers.3.self_attn.q_norm.weight")
    names = ["model.embed_tokens.weight", "model.norm.weight", "lm_head.weight", "model.rotary.inv_freq"] + \
        [f"model.layers.{i}.mlp.down_proj.weight" for i in range(6)]
    assert "model.rotary.inv_freq" not in ad.convert_weight_name_meta(names)
    # 8 layer slots over 3 stages, slots 2 and 5 are no-ops: real layers 0..5 sit in slots 0,1,3,4,6,7
    per = ad.get_weight_names_per_pp([3, 3, 2], ad.convert_weight_name_meta(names), noop_layers=[2, 5])
    assert per[0][:1] == ["model.embed_tokens.weight"] and per[2][:2] == ["model.norm.weight", "lm_head.weight"]
    assert [ad.layer_of(n) for n in per[0][1:]] == [0, 1] and [ad.layer_of(n) for n in per[1]] == [2, 3]
    assert ad.global2local_layer("model.layers.4.mlp.down_proj.weight", [3, 3, 2], [2, 5]) == \
        (2, "model.layers.0.mlp.down_proj.weight")
    mla = get_weight_adaptor("DeepseekV3ForCausalLM")
    assert mla.replace_name_i2t("model.layers.5.self_attn.kv_b_proj.weight").endswith("linear_kv_up_proj.weight")
    with pytest.raises(ValueError):
        get_weight_adaptor("NoSuchModel")


def test_optimizer_config_builds_optimizer_and_schedule():
    from types import SimpleNamespace

    from mindspeed_rl_b200.parallel.ddp import DistributedDataParallel
    cfg = SimpleNamespace(lr=2e-3, min_lr=2e-4, weight_decay=0.05, adam_beta2=0.95, clip_grad=0.5, bf16=True,
                          lr_decay_style="cosine", lr_warmup_iters=2, train_iters=10, reuse_fp32_param=True,
                          unknown_knob=1)
    oc = OptimizerConfig.from_training_config(cfg)
    assert oc.params_dtype == torch.bfloat16 and oc.adam_beta1 == 0.9 and oc.adam_beta2 == 0.95
    m = DistributedDataParallel(torch.nn.Linear(16, 16, bias=False).bfloat16())
    opt, sched = oc.build(m.buffers)
    assert opt.reuse_fp32_param and opt.clip_grad == 0.5 and opt.param_groups[0]["weight_decay"] == 0.05
    lrs = []
    for _ in range(10):
        sched.step()
        lrs.append(opt.param_groups[0]["lr"])
    assert lrs[1] == pytest.approx(2e-3) and lrs[-1] == pytest.approx(2e-4) and lrs[0] < lrs[1] > lrs[5] > lrs[-1]
    with pytest.raises(ValueError):
        OptimizerConfig.from_training_config(dict(optimizer="sgd"))


def test_engine_implements_the_contract():
    assert issubclass(LLMEngine, BaseInferEngine)
    for name in ("init_cache_engine", "free_cache_engine", "offload_model_weights", "sync_model_weights",
                 "generate_sequences"):
        assert getattr(LLMEngine, name) is not getattr(BaseInferEngine, name)
