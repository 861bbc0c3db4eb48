"""Training-backend configuration (``MegatronConfig``).

Holds every knob the YAML sections ``megatron_training`` / ``actor_config`` /
``ref_config`` / ``reward_config`` / ``critic_config`` and the ``model`` catalogue may set.
Key names and defaults follow the reference's ``MegatronConfig``
(``mindspeed_rl/config_cls/megatron_config.py:199-385``) so existing YAML files load
unchanged; here they are organised as schema groups consumed by our own backend.
"""
from __future__ import annotations

import os

from .schema import SchemaConfig, merge_schemas

TEMPLATES_DIR = os.path.abspath(
    os.path.join(os.path.dirname(__file__), "..", "..", "configs", "model", "templates.json")
)

# --- model architecture -------------------------------------------------------------
ARCH = dict(
    use_mcore_models=False, spec=None, transformer_impl="local",
    num_layers=None, hidden_size=None, ffn_hidden_size=None, num_attention_heads=None,
    kv_channels=None, group_query_attention=False, num_query_groups=1,
    untie_embeddings_and_output_weights=False, qk_layernorm=False,
    add_qkv_bias=False, disable_bias_linear=False, attention_bias=False,
    attention_dropout=0.1, hidden_dropout=0.1, init_method_std=0.02,
    position_embedding_type="learned_absolute", use_rotary_position_embeddings=False,
    rotary_base=10000, max_position_embeddings=None,
    normalization="LayerNorm", norm_epsilon=1e-5, swiglu=False,
    make_vocab_size_divisible_by=128, padded_vocab_size=None, vocab_extra_ids=0,
    shape_order="SBH", attention_mask_type="causal", attention_softmax_in_fp32=False,
    mm_model=None,
)

# --- RoPE scaling (YaRN / llama3) ---------------------------------------------------
ROPE_SCALING = dict(
    rope_scaling_type=None, rope_scaling_factor=1.0, low_freq_factor=None,
    high_freq_factor=None, original_max_position_embeddings=None,
    beta_fast=32, beta_slow=1, rope_scaling_mscale=1.0, rope_scaling_mscale_all_dim=0.0,
    rope_scaling_original_max_position_embeddings=None,
)

# --- multi-latent attention ---------------------------------------------------------
MLA = dict(
    multi_latent_attention=False, qk_pos_emb_head_dim=None, qk_head_dim=None,
    q_lora_rank=None, kv_lora_rank=None, v_head_dim=None,
)

# --- vision-language models ----------------------------------------------------------
VISION = dict(
    image_token_id=151655, video_token_id=151656, vision_start_token_id=151652, vision_end_token_id=151653,
    patch_size=14, spatial_merge_size=2, mrope_section=None,
)

# --- mixture of experts -------------------------------------------------------------
MOE = dict(
    num_experts=None, moe_router_topk=2, moe_ffn_hidden_size=None, n_shared_experts=None,
    moe_grouped_gemm=False, moe_permutation_async_comm=False, moe_tp_extend_ep=False,
    moe_alltoall_overlap_comm=False, use_fused_moe_token_permute_and_unpermute=False,
    moe_token_dispatcher_type=None, moe_p2p_capacity_factor=0.0, seq_aux=False, first_k_dense_replace=None,
    moe_layer_freq=None, moe_router_load_balancing_type="aux_loss",
    moe_router_num_groups=None, moe_router_group_topk=None,
    moe_router_topk_scaling_factor=None, norm_topk_prob=False,
    moe_router_score_function="softmax", moe_router_enable_expert_bias=False,
    moe_aux_loss_coeff=0.001,
)

# --- fused-kernel switches (all map onto our sm_100a kernels) -----------------------
FUSION = dict(
    use_flash_attn=False, use_fused_rmsnorm=False, use_fused_swiglu=False,
    use_fused_rotary_pos_emb=False, no_bias_dropout_fusion=False,
    no_masked_softmax_fusion=False, no_gradient_accumulation_fusion=False,
    gemm_gradient_accumulation_fusion=False, use_fused_ring_attention_update=False,
    use_ascend_coc=False, coc_mode=-1, coc_parallel_num=1, coc_fused_kernel=False,
)

# --- parallelism --------------------------------------------------------------------
PARALLEL = dict(
    tensor_model_parallel_size=1, pipeline_model_parallel_size=1,
    expert_model_parallel_size=1, context_parallel_size=1,
    context_parallel_algo="ulysses_cp_algo", ulysses_degree_in_cp=None, sequence_parallel=False,
    num_layers_per_virtual_pipeline_stage=None, num_layer_list=None, noop_layers=None,
    use_tp_pp_dp_mapping=False, use_cp_send_recv_overlap=False,
    use_distributed_optimizer=False, overlap_grad_reduce=False, overlap_param_gather=False,
    ddp_bucket_size=None, accumulate_allreduce_grads_in_fp32=False,
    distributed_backend="nccl",
)

# --- optimisation -------------------------------------------------------------------
OPTIM = dict(
    optimizer="adam", lr=None, min_lr=0.0, lr_decay_style="linear", lr_warmup_fraction=None,
    weight_decay=0.01, clip_grad=1.0, adam_beta1=0.9, adam_beta2=0.999,
    initial_loss_scale=2 ** 32, bf16=True, no_check_for_nan_in_loss_and_grad=False,
    reuse_fp32_param=False, swap_optimizer=False,
)

# --- memory -------------------------------------------------------------------------
MEMORY = dict(
    recompute_granularity=None, recompute_method=None, recompute_num_layers=None,
    recompute_activation_function=False, swap_attention=False,
    # accepted for recipe compatibility; both savings are built into the kernels' backward passes
    # (the norm backward rebuilds the normalised rows, the SwiGLU backward rebuilds silu(g)*u)
    recompute_activation_function_num_layers=None, recompute_norm=False, recompute_norm_num_layers=None,
    swap_modules="input_norm,self_attention,post_attention_norm",
)

# --- batches, data, run control -----------------------------------------------------
RUN = dict(
    global_batch_size=None, micro_batch_size=None, seq_length=None, train_iters=None,
    eval_iters=100, eval_interval=1000, log_interval=100, log_throughput=False,
    skip_train=False, seed=1234, stage=None, algorithm=None, ai_framework=None,
    npu_deterministic=False, use_deterministic=False, enable_high_availability=False,
    tokenizer_type=None, tokenizer_name_or_path=None, tokenizer_not_use_fast=False,
    tokenizer_padding_side="right", prompt_type=None, prompt_type_path=TEMPLATES_DIR,
    data_path=None, split=None, dataloader_type=None, num_workers=2,
    is_instruction_dataset=False, is_pairwise_dataset=False,
    full_shuffle_instruction_dataset=False, no_shuffle=False, dataset_additional_keys=[],
    variable_seq_lengths=False, no_pad_to_seq_lengths=False, pad_to_multiple_of=8,
    reset_position_ids=False, reset_attention_mask=False,
    do_sample=False, use_kv_cache=False,
)

# --- checkpointing ------------------------------------------------------------------
CKPT = dict(
    load=None, save=None, save_interval=None, finetune=False, pretrained_checkpoint=None,
    no_load_optim=None, no_load_rng=None, no_save_optim=None, no_save_rng=None,
    no_shared_storage=False, load_checkpoint_loosely=False,
)

# --- LoRA / DPO ---------------------------------------------------------------------
ADAPT = dict(
    lora_ckpt_filter=False, lora_r=8, lora_alpha=16, lora_fusion=False,
    lora_target_modules=None,
    dpo_loss_type="sigmoid", dpo_beta=0.1, dpo_label_smoothing=0.0, ref_model="", refer_model_iter=1,
)


def _int_list(value, key: str):
    """``"16,17,16,15"`` / ``[16, 17]`` / ``7`` -> list of ints; ``None`` and ``""`` stay ``None``."""
    if value is None or value == "":
        return None
    if isinstance(value, str):
        value = [v for v in value.replace(" ", "").split(",") if v]
    elif isinstance(value, int):
        value = [value]
    if any(isinstance(v, (list, tuple)) for v in value):
        # vision-language models: [layers of the vision tower per stage, layers of the decoder per stage]
        return [_int_list(v, key) if isinstance(v, (list, tuple)) else [int(v)] for v in value]
    try:
        return [int(v) for v in value]
    except (TypeError, ValueError):
        raise ValueError(f"{key}: expected comma-separated integers, got {value!r}") from None


class MegatronConfig(SchemaConfig):
    """Flat training config built from a role dict layered over a model dict.

    ``MegatronConfig(training_dict, model_catalogue)``: when ``training_dict`` contains
    ``model: <name>``, ``model_catalogue[name]`` is applied first and the role keys
    override it.  ``pad_to_multiple_of`` is forced to ``tp * cp`` afterwards
    (reference: ``megatron_config.py:381-385``).
    """

    SCHEMA = merge_schemas(ARCH, ROPE_SCALING, MLA, VISION, MOE, FUSION, PARALLEL, OPTIM, MEMORY, RUN,
                           CKPT, ADAPT)

    def __init__(self, training_config=None, model_config=None):
        self._model_catalogue = model_config
        super().__init__(training_config)

    def _extra_init(self, **kw):
        pass

    def update(self, config_dict, model_config_dict=None):
        if model_config_dict is None and "model" in config_dict:
            model_config_dict = self.__dict__.get("_model_catalogue")
        super().update(config_dict, model_config_dict)

    def _finalize(self):
        self.__dict__.pop("_model_catalogue", None)
        self.pad_to_multiple_of = self.tensor_model_parallel_size * self.context_parallel_size
        # recipes write per-stage layer counts and empty slots as "16,17,16,15"
        for key in ("num_layer_list", "noop_layers"):
            self.__dict__[key] = _int_list(self.__dict__.get(key), key)

    # convenience accessors used by the backend ---------------------------------------
    @property
    def head_dim(self) -> int:
        return self.kv_channels or (self.hidden_size // self.num_attention_heads)

    @property
    def num_kv_heads(self) -> int:
        return self.num_query_groups if self.group_query_attention else self.num_attention_heads
