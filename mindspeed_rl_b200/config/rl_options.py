"""RL-level, rollout-engine, profiler, dump-tool and dataset-preprocessing configs.

YAML sections: ``rl_config`` -> :class:`RLConfig`, ``generate_config`` ->
:class:`GenerateConfig`, ``profiler_config.<role>`` -> :class:`ProfilerConfig`,
``msprobe_config`` -> :class:`MsprobeConfig`, dataset YAMLs -> :class:`DataHandlerConfig`.
Key names and defaults match the reference (``mindspeed_rl/config_cls/rl_config.py:122-255``,
``generate_config.py:49-105``, ``mindstudio_config.py:6-102``,
``data_handler_config.py:15-132``); ``num_gpus`` is accepted as an alias of ``num_npus`` in
every ``*_resource`` block.
"""
from __future__ import annotations

import os

from .schema import ConfigKeyError, SchemaConfig, merge_schemas
from .training_config import TEMPLATES_DIR

# ---------------------------------------------------------------------------------------
# RLConfig
# ---------------------------------------------------------------------------------------
_RESOURCES = dict(
    runtime_env_path="configs/envs/runtime_env.yaml", hccl_buffersize=256,
    actor_resource={"num_npus": None}, reference_resource=None, reward_resource=None,
    critic_resource=None, vit_resource=None, integrated_mode_config=None,
    use_integrated_worker=True, colocate_actor_and_vit=False,
    num_cpus_for_local_task=1, num_cpus_for_placement_group=8,
)

_ALGO = dict(
    rule_reward=True, beta=0.1, num_samples_per_step=1, max_prompt_length=512, epochs=1,
    clip_ratio=0.2, cliprange_value=0.5, entropy_coeff=0.0, gamma=1.0, lam=0.95,
    advantage_whiten=True, kl_penalty="low_var_kl", kl_ctrl_type="fixed", init_kl_coef=0.01,
    kl_horizon=1000, kl_target=100.0, adv_estimator="group_norm",
    verifier_function=["base_acc"], verifier_weight=[1.0], verifier_parallel=1,
    verifier_timeout=30, use_kl_in_reward=False, shuffle_mini_batch=False,
    tp_split_expert=False, n_samples_per_prompt=1, mini_batch_size=1, token_level_loss=True,
    share_backbone=False,
)

_LOGGING = dict(
    use_tensorboard=False, use_wandb=False, wandb_project="", wandb_exp_name="",
    wandb_save_dir="", use_swanlab=False, swanlab_mode="", swanlab_project="",
    swanlab_exp_name="", swanlab_save_dir="", log_max_throughput=True,
)

_SCHEDULING = dict(
    blocking=True, async_engine=False, guarantee_order=False, use_dp_batch_balance=False,
    ref_forward_micro_batch_size=None, actor_forward_micro_batch_size=None,
    vit_forward_micro_batch_size=None,
    actor_rollout_dispatch_size=None, actor_logprob_dispatch_size=None, ref_dispatch_size=None,
    reward_dispatch_size=None, dynamic_sampling_dispatch_size=None, adv_dispatch_size=None,
    actor_update_dispatch_size=None, critic_update_dispatch_size=None,
    critic_value_dispatch_size=None, kl_dispatch_size=None,
    actor_image_embeds_dispatch_size=None,
    data_strategy="td", transfer_queue_data_shard_num=1,
    transfer_queue_data_shard_port_base=None, zmq_communication=True,
)

_PACKING = dict(
    is_multimodal=False, use_remove_padding=False, reuse_image_embeds=False,
    use_dynamic_bsz=False, max_packing_token_size=4096,
    ref_max_packing_token_size=None, actor_max_packing_token_size=None,
    update_max_packing_token_size=None, dynamic_max_batch_size=None,
    ref_dynamic_max_batch_size=None, actor_dynamic_max_batch_size=None,
    update_dynamic_max_batch_size=None,
)

_DAPO = dict(
    clip_higher_enable=False, clip_ratio_low=0.1, clip_ratio_high=0.1,
    overlong_buffer_enable=False, overlong_buffer=0, overlong_buffer_penalty_factor=1.0,
    rollout_max_tokens=2048, filter_groups_enable=False, filter_groups_metric="acc",
    filter_groups_max_batches=1, filter_groups_train_batch_size=1,
)

_ROLLOUT_FLOW = dict(
    partial_rollout_max_split=1, require_max_age_all_finished=True,
    multi_turn_enable=False, tool_config_path=None, max_tool_calls=0, max_parallel_calls=0,
    max_total_response_length=0, max_tool_response_length=0,
    tool_response_truncate_side=None, tool_parser_format=None,
)

_RESOURCE_KEYS = ("actor_resource", "reference_resource", "reward_resource", "critic_resource",
                  "vit_resource")


def _normalise_resource(block):
    """Accept ``num_gpus`` for ``num_npus`` and reject anything else."""
    if block is None:
        return None
    out = {}
    for k, v in dict(block).items():
        k2 = "num_npus" if k == "num_gpus" else k
        if k2 != "num_npus":
            raise ConfigKeyError(f"resource block: unknown key '{k}' (expected num_npus/num_gpus)")
        out[k2] = v
    return out


class RLConfig(SchemaConfig):
    """All algorithm / scheduling / logging options of an RL run (``rl_config``)."""

    SCHEMA = merge_schemas(_RESOURCES, _ALGO, _LOGGING, _SCHEDULING, _PACKING, _DAPO,
                           _ROLLOUT_FLOW)

    def __init__(self, config_dict=None):
        super().__init__(config_dict or {})

    def update(self, config_dict, model_config_dict=None):
        cfg = dict(config_dict)
        for key in _RESOURCE_KEYS:
            if cfg.get(key) is not None:
                cfg[key] = _normalise_resource(cfg[key])
        super().update(cfg)

    def _finalize(self):
        # mini_batch_size is given in prompts; internally it counts samples
        # (reference: rl_config.py:256)
        self.mini_batch_size = self.mini_batch_size * self.n_samples_per_prompt
        # per-stage packing sizes inherit the common value unless given explicitly
        for stage in ("ref", "actor", "update"):
            if getattr(self, f"{stage}_max_packing_token_size") is None:
                setattr(self, f"{stage}_max_packing_token_size", self.max_packing_token_size)
            if getattr(self, f"{stage}_dynamic_max_batch_size") is None:
                setattr(self, f"{stage}_dynamic_max_batch_size", self.dynamic_max_batch_size)

    @property
    def num_gpus(self):
        return (self.actor_resource or {}).get("num_npus")


# ---------------------------------------------------------------------------------------
# GenerateConfig
# ---------------------------------------------------------------------------------------
_SAMPLING_DEFAULTS = {
    "logprobs": 1, "max_tokens": 128, "top_p": 1.0, "top_k": 50, "min_p": 0.0,
    "temperature": 0.2, "detokenize": False, "seed": None,
}

_GENERATE = dict(
    limit_mm_image_per_prompt=1, limit_mm_video_per_prompt=0,
    data_parallel_size=None, tokenizer_name_or_path="/path/to/tokenizer",
    trust_remote_code=False,
    eplb_token_collects=False, eplb_token_save_path="./", expert_map_path=None,
    infer_tensor_parallel_size=8, infer_pipeline_parallel_size=1,
    infer_expert_parallel_size=1,
    max_num_seqs=1, max_model_len=2048, max_num_batched_tokens=2048, dtype="bfloat16",
    gpu_memory_utilization=0.5, offload_train_optimizer=False, offload_train_grad=False,
    offload_train_param=False,
    enable_prefix_caching=False, num_scheduler_steps=1, enforce_eager=True,
    torchair_graph=False, enable_expert_parallel=False, ascend_scheduler_config_enabled=True,
    sampling_config=_SAMPLING_DEFAULTS,
    # B200 additions (all optional): block size of the paged KV cache, fp8 block-scaled
    # rollout GEMM weights, CUDA-graph decode buckets.
    kv_block_size=16, rollout_fp8=False,
    graph_batch_sizes=[8, 16, 32, 64, 128, 192, 256, 384, 512],
)


class GenerateConfig(SchemaConfig):
    """Rollout-engine options (``generate_config``)."""

    SCHEMA = _GENERATE

    def __init__(self, config_dict=None):
        super().__init__(config_dict or {})

    def update(self, config_dict, model_config_dict=None):
        cfg = dict(config_dict)
        sampling = cfg.pop("sampling_config", None)
        super().update(cfg)
        if sampling is not None:
            merged = dict(self.sampling_config)
            for k, v in sampling.items():
                if k not in _SAMPLING_DEFAULTS:
                    raise ConfigKeyError(f"sampling_config: unknown key '{k}'")
                merged[k] = v
            self.sampling_config = merged


# ---------------------------------------------------------------------------------------
# Profiler / dump tool
# ---------------------------------------------------------------------------------------
class ProfilerConfig(SchemaConfig):
    """``profiler_config.<role>``: which stage / steps / ranks to trace and how."""

    SCHEMA = dict(
        profile=False, mstx=False, stage="all", profile_save_path="",
        profile_export_type="text", profile_level="level0", profile_with_memory=False,
        profile_record_shapes=False, profile_with_cpu=True, profile_with_npu=True,
        profile_with_module=False, profile_step_start=1, profile_step_end=2,
        profile_analysis=False, profile_ranks="all",
    )

    def __init__(self, config_dict=None, role=""):
        self.role = role
        super().__init__(config_dict or {})

    def _extra_init(self, **kw):
        pass


class MsprobeConfig(SchemaConfig):
    """``msprobe_config``: tensor / configuration dump switches per stage and step range."""

    SCHEMA = dict(
        msprobe=False, dump_path="./msprobe_dump", key_data_dump=False,
        configurations_dump=False, actor_train_dump=False, actor_infer_dump=False,
        token_range_start=0, token_range_end=0, reference_dump=False, critic_train_dump=False,
        step_start=0, step_end=0,
    )

    def __init__(self, config_dict=None, role=""):
        self.role = role
        super().__init__(config_dict or {})

    def _extra_init(self, **kw):
        pass


# ---------------------------------------------------------------------------------------
# Dataset preprocessing
# ---------------------------------------------------------------------------------------
class DataHandlerConfig(SchemaConfig):
    """Options of ``cli/preprocess_data.py`` (raw json/parquet -> tokenised .bin/.idx)."""

    SCHEMA = dict(
        input=None, handler_name="", streaming=False, json_keys=["text"],
        split_sentences=False, keep_newlines=False, prompt_type="empty",
        prompt_type_path=TEMPLATES_DIR, dataset_additional_keys=[], interleave_probs=None,
        overwrite_cache=False, seed=1234,
        cache_dir=os.path.join(os.path.expanduser("~"), "cache"), map_keys=None, pack=False,
        neat_pack=False, script_data_dir=None, tokenizer_type="HuggingFaceTokenizer",
        tokenizer_not_use_fast=True, vocab_file=None, merge_file=None, append_eod=False,
        tokenizer_name_or_path=None, seq_length=None, make_vocab_size_divisible_by=128,
        pad_vocab_size_to=None, placeholder_token="ки", reward_tokens=[], output_prefix=None,
        dataset_impl="mmap", workers=1, n_subs=1, log_interval=100, merge_group_keys=None,
        enable_thinking=False,
    )

    def __init__(self, config_dict=None):
        super().__init__(config_dict or {})

    def _finalize(self):
        if self.input is None:
            raise ValueError("DataHandlerConfig: 'input' is required")
        if self.output_prefix is None:
            raise ValueError("DataHandlerConfig: 'output_prefix' is required")
        if self.workers < 1 or self.n_subs < 1:
            raise ValueError("DataHandlerConfig: workers and n_subs must be >= 1")
        if self.workers % self.n_subs != 0:
            raise ValueError("DataHandlerConfig: workers must be a multiple of n_subs")
