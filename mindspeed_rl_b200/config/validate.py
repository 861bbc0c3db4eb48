"""Cross-section validation and derivation of the per-stage dispatch sizes.

``validate_rl_args`` enforces the same rules and fills the same derived fields as the
reference validator (``mindspeed_rl/config_cls/validate_config.py:9-519``): bf16 only,
integrated-worker constraints, ``max_model_len >= seq_length``, CP / remove-padding
constraints, resource divisibility, batch divisibility, rollout DP derivation, default
``*_dispatch_size`` values and their bounds, DAPO / partial-rollout / multi-turn checks.
The rules are expressed as small composable checks over a ``_Layout`` record per role.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

from .rl_options import GenerateConfig, RLConfig
from .training_config import MegatronConfig

_CP_ALGOS = ("ulysses_cp_algo", "megatron_cp_algo", "hybrid_cp_algo")


def get_node_nums() -> int:
    """Number of nodes that host CPU-side reward actors.

    With Ray this is the number of alive nodes; the local runtime runs on one node.
    ``MSRL_NUM_NODES`` overrides the detection (useful in tests).
    """
    env = os.environ.get("MSRL_NUM_NODES")
    if env:
        return max(1, int(env))
    try:  # pragma: no cover - ray is optional
        import ray

        if ray.is_initialized():
            return max(1, len([n for n in ray.nodes() if n.get("Alive")]))
    except Exception:
        pass
    return 1


@dataclass
class _Layout:
    name: str
    gpus: int
    tp: int
    pp: int
    cp: int
    gbs: int
    mbs: int

    @property
    def model_parallel(self) -> int:
        return self.tp * self.pp * self.cp

    @property
    def dp(self) -> int:
        return self.gpus // self.model_parallel


def _layout(name: str, cfg: MegatronConfig, resource) -> _Layout:
    return _Layout(name, resource["num_npus"], cfg.tensor_model_parallel_size,
                   cfg.pipeline_model_parallel_size, cfg.context_parallel_size,
                   cfg.global_batch_size, cfg.micro_batch_size)


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise ValueError(msg)


def _check_resource(lay: _Layout) -> None:
    _require(lay.gpus % lay.model_parallel == 0,
             f"{lay.name}: {lay.gpus} devices are not divisible by tp*pp*cp = "
             f"{lay.tp}*{lay.pp}*{lay.cp} = {lay.model_parallel}")


def _check_batch(lay: _Layout, n: int) -> None:
    _require((lay.gbs * n) % lay.mbs == 0,
             f"{lay.name}: global_batch_size*n_samples = {lay.gbs * n} must be divisible by "
             f"micro_batch_size {lay.mbs}")


def _check_dp_batch(name: str, gbs: int, dp: int, mbs: int, n: int) -> None:
    _require(dp > 0 and gbs % dp == 0,
             f"{name}: global_batch_size {gbs} must be divisible by data_parallel_size {dp}")
    _require((gbs // dp * n) % mbs == 0,
             f"{name}: (global_batch_size // dp) * n_samples = {gbs // dp * n} must be "
             f"divisible by {mbs}")


def _check_divides(name: str, gbs: int, n: int, dispatch: int) -> None:
    _require(dispatch and (gbs * n) % dispatch == 0,
             f"{name}: global_batch_size*n_samples = {gbs * n} must be divisible by the "
             f"dispatch size {dispatch}")


def _check_dispatch_bound(name: str, dispatch: Optional[int], gbs: int, n: int, dp: int) -> None:
    if dispatch and dispatch > gbs * n // dp:
        raise ValueError(f"{name} = {dispatch} exceeds the samples available per data-parallel "
                         f"rank ({gbs}*{n}//{dp} = {gbs * n // dp})")


def validate_rl_args(actor_config: MegatronConfig, ref_config: Optional[MegatronConfig],
                     reward_config: MegatronConfig, rl_config: RLConfig,
                     generate_config: GenerateConfig,
                     critic_config: Optional[MegatronConfig] = None,
                     vit_config: Optional[MegatronConfig] = None) -> None:
    rl, gen = rl_config, generate_config
    n = rl.n_samples_per_prompt

    # -- framework / dtype ---------------------------------------------------------------
    fw = getattr(actor_config, "ai_framework", None)
    _require(fw in (None, "mindspore"), f"ai_framework '{fw}' is not supported (None|mindspore)")
    _require(fw is None, "ai_framework: mindspore is outside the scope of the B200 build")
    _require(actor_config.bf16 is not False and gen.dtype == "bfloat16",
             "bf16 must be true and generate_config.dtype must be bfloat16")

    # -- tied embeddings need the first and last pipeline stage to share one gradient --------
    for name, cfg in (("Actor", actor_config), ("Reference", ref_config), ("Critic", critic_config)):
        if cfg is None:
            continue
        tied = getattr(cfg, "untie_embeddings_and_output_weights", True) is False
        _require(not (tied and (cfg.pipeline_model_parallel_size or 1) > 1),
                 f"{name}: tied input/output embeddings are not supported with pipeline_model_parallel_size > 1 "
                 f"(the two stages' copies would drift apart); set untie_embeddings_and_output_weights: true")

    # -- co-location ----------------------------------------------------------------------
    if rl.use_integrated_worker:
        _require(rl.reference_resource is None,
                 "reference_resource must not be set when use_integrated_worker is on")
        rl.reference_resource = rl.actor_resource
        _require(rl.reward_resource is None,
                 "a reward model is not supported when use_integrated_worker is on")
    else:
        _require(rl.integrated_mode_config is None,
                 "integrated_mode_config must not be set when use_integrated_worker is off")

    # -- what the parallel sizes have to divide ---------------------------------------------
    a = actor_config
    if getattr(a, "num_attention_heads", None):
        kv_heads = a.num_query_groups if a.group_query_attention else a.num_attention_heads
        for label, tp in (("tensor_model_parallel_size", a.tensor_model_parallel_size or 1),
                          ("infer_tensor_parallel_size", gen.infer_tensor_parallel_size or 1)):
            _require(a.num_attention_heads % tp == 0,
                     f"{label} {tp} must divide the {a.num_attention_heads} attention heads")
            _require(a.multi_latent_attention or kv_heads % tp == 0,
                     f"{label} {tp} must divide the {kv_heads} key / value heads")
            _require(not a.padded_vocab_size or a.padded_vocab_size % tp == 0,
                     f"{label} {tp} must divide the padded vocabulary size {a.padded_vocab_size}")
    if getattr(a, "num_experts", None):
        tp, ep = a.tensor_model_parallel_size or 1, a.expert_model_parallel_size or 1
        _require(not (tp > 1 and ep > 1) or a.moe_tp_extend_ep,
                 "expert models with tensor_model_parallel_size > 1 and expert_model_parallel_size > 1 need "
                 "moe_tp_extend_ep (experts are spread over TP x EP, never cut by TP)")
        _require(not (tp > 1 and a.moe_tp_extend_ep) or a.sequence_parallel,
                 "moe_tp_extend_ep with tensor parallelism needs sequence_parallel")
        spread = ep * tp if a.moe_tp_extend_ep else ep
        _require(a.num_experts % spread == 0,
                 f"{a.num_experts} experts do not divide over {spread} training expert-parallel ranks")
        infer_ep = gen.infer_expert_parallel_size or 1
        _require(a.num_experts % infer_ep == 0 or bool(getattr(gen, "expert_map_path", None)),
                 f"{a.num_experts} experts do not divide over infer_expert_parallel_size {infer_ep}")

    # -- lengths, CP, packing -------------------------------------------------------------
    _require(gen.max_model_len >= actor_config.seq_length,
             f"seq_length {actor_config.seq_length} exceeds generate_config.max_model_len "
             f"{gen.max_model_len}")
    ring_cp = False
    if actor_config.context_parallel_size > 1 and actor_config.context_parallel_algo is not None:
        _require(actor_config.context_parallel_algo in _CP_ALGOS,
                 f"context_parallel_algo must be one of {_CP_ALGOS}")
        ring_cp = actor_config.context_parallel_algo == "megatron_cp_algo"
    if ring_cp and rl.use_remove_padding:
        _require(actor_config.reset_attention_mask,
                 "ring context parallel with remove-padding needs reset_attention_mask=true")
    if rl.use_remove_padding:
        _require(actor_config.pipeline_model_parallel_size == 1
                 or actor_config.no_pad_to_seq_lengths,
                 "use_remove_padding with pipeline parallelism needs no_pad_to_seq_lengths=true")
        _require(actor_config.reset_attention_mask,
                 "use_remove_padding needs reset_attention_mask=true")
        _require(not rl.is_multimodal, "multimodal models cannot use use_remove_padding")

    # -- resources and batches -------------------------------------------------------------
    actor = _layout("Actor", actor_config, rl.actor_resource)
    _check_resource(actor)
    ref = None
    if ref_config:
        ref = _layout("Reference", ref_config, rl.reference_resource)
        _check_resource(ref)
    reward = None
    if rl.reward_resource:
        reward = _layout("Reward", reward_config, rl.reward_resource)
        _check_resource(reward)
    critic = None
    if rl.critic_resource:
        critic = _layout("Critic", critic_config, rl.critic_resource)
    vit = None
    if rl.colocate_actor_and_vit:
        vit = _layout("Vit", vit_config, rl.vit_resource)

    _check_batch(actor, n)
    if ref:
        _check_batch(ref, n)
    if reward:
        _check_batch(reward, n)

    _require(gen.infer_pipeline_parallel_size == 1,
             "pipeline parallel rollout is not supported (infer_pipeline_parallel_size must be 1)")
    gen.data_parallel_size = actor.gpus // (gen.infer_tensor_parallel_size
                                            * gen.infer_pipeline_parallel_size)
    rollout_dp = gen.data_parallel_size

    _check_dp_batch("Actor", actor.gbs, actor.dp, actor.mbs, n)
    rl.actor_rollout_dispatch_size = rl.actor_rollout_dispatch_size or actor.gbs * n // rollout_dp
    _check_dp_batch("Generation", actor.gbs, rollout_dp, rl.actor_rollout_dispatch_size, n)
    if not rl.use_integrated_worker and ref:
        _check_dp_batch("Reference", ref.gbs, ref.dp, ref.mbs, n)
    if reward and not rl.use_integrated_worker:
        _check_dp_batch("Reward", reward.gbs, reward.dp, reward.mbs, n)

    # -- default dispatch sizes --------------------------------------------------------------
    nodes = get_node_nums()
    train_gbs = rl.filter_groups_train_batch_size if rl.filter_groups_enable else actor.gbs
    if rl.filter_groups_enable:
        _check_dp_batch("ActorForDapo", train_gbs, actor.dp, actor.mbs, n)
        rl.dynamic_sampling_dispatch_size = (rl.dynamic_sampling_dispatch_size
                                             or reward_config.global_batch_size * n // nodes)
    rl.actor_logprob_dispatch_size = rl.actor_logprob_dispatch_size or train_gbs * n // actor.dp
    rl.adv_dispatch_size = rl.adv_dispatch_size or train_gbs * n
    if ref:
        rl.ref_dispatch_size = rl.ref_dispatch_size or ref.gbs * n // ref.dp
    if rl.reuse_image_embeds:
        src = vit if vit else actor
        rl.actor_image_embeds_dispatch_size = (rl.actor_image_embeds_dispatch_size
                                               or src.gbs * n // src.dp)
    if reward:
        rl.reward_dispatch_size = rl.reward_dispatch_size or reward.gbs * n // reward.dp
    else:
        rl.reward_dispatch_size = (rl.reward_dispatch_size
                                   or reward_config.global_batch_size * n // nodes)
        _require(reward_config.global_batch_size % nodes == 0,
                 f"global_batch_size {reward_config.global_batch_size} must be divisible by the "
                 f"number of nodes ({nodes}) hosting rule-reward actors")

    if rl.share_backbone:
        _require(bool(actor_config.lora_target_modules),
                 "share_backbone can only be used together with LoRA")
        _require(actor_config.stage != "ray_dapo", "share_backbone is not available for ray_dapo")

    if critic:
        rl.critic_update_dispatch_size = rl.critic_update_dispatch_size or critic.gbs * n // critic.dp
        rl.critic_value_dispatch_size = rl.critic_value_dispatch_size or critic.gbs * n // critic.dp
        rl.kl_dispatch_size = rl.kl_dispatch_size or critic.gbs * n

    # -- dispatch sizes divide the batch ---------------------------------------------------------
    _check_divides("Actor Infer", train_gbs, n, rl.actor_logprob_dispatch_size)
    _check_divides("Advantages", train_gbs, n, rl.adv_dispatch_size)
    if rl.filter_groups_enable:
        _check_divides("Dynamic Sampling", reward_config.global_batch_size, n,
                       rl.dynamic_sampling_dispatch_size)
        _require(rl.dynamic_sampling_dispatch_size % n == 0,
                 "dynamic_sampling_dispatch_size must be a multiple of n_samples_per_prompt")
    if ref:
        _check_divides("Reference", ref.gbs, n, rl.ref_dispatch_size)
    _check_divides("Reward" if reward else "Rule Reward", reward_config.global_batch_size, n,
                   rl.reward_dispatch_size)
    if critic:
        _check_divides("Critic Infer", critic.gbs, n, rl.critic_value_dispatch_size)
        _check_divides("KL", critic.gbs, n, rl.kl_dispatch_size)
        _check_divides("Critic Update", critic.gbs, n, rl.critic_update_dispatch_size)

    # -- user-given sizes stay within the per-DP share --------------------------------------------
    if rl.actor_update_dispatch_size:
        _require(rl.actor_update_dispatch_size >= rl.mini_batch_size / actor.dp,
                 f"actor_update_dispatch_size {rl.actor_update_dispatch_size} must be >= "
                 f"mini_batch_size/dp = {rl.mini_batch_size}/{actor.dp}")
    _check_dispatch_bound("actor_rollout_dispatch_size", rl.actor_rollout_dispatch_size,
                          actor.gbs, n, rollout_dp)
    _check_dispatch_bound("actor_logprob_dispatch_size", rl.actor_logprob_dispatch_size,
                          actor.gbs, n, actor.dp)
    if ref:
        _check_dispatch_bound("ref_dispatch_size", rl.ref_dispatch_size, ref.gbs, n, ref.dp)
    _check_dispatch_bound("actor_update_dispatch_size", rl.actor_update_dispatch_size,
                          actor.gbs, n, actor.dp)
    if critic:
        _check_dispatch_bound("critic_update_dispatch_size", rl.critic_update_dispatch_size,
                              critic.gbs, n, critic.dp)
        _check_dispatch_bound("critic_value_dispatch_size", rl.critic_value_dispatch_size,
                              critic.gbs, n, critic.dp)
        _check_dispatch_bound("kl_dispatch_size", rl.kl_dispatch_size, critic.gbs, n, 1)
    if reward:
        _check_dispatch_bound("reward_dispatch_size", rl.reward_dispatch_size, reward.gbs, n,
                              reward.dp)
    _check_dispatch_bound("dynamic_sampling_dispatch_size", rl.dynamic_sampling_dispatch_size,
                          reward_config.global_batch_size, n, nodes)
    if rl.reuse_image_embeds:
        _check_dispatch_bound("actor_image_embeds_dispatch_size",
                              rl.actor_image_embeds_dispatch_size, actor.gbs, n, actor.dp)
        if vit:
            _check_dispatch_bound("actor_image_embeds_dispatch_size",
                                  rl.actor_image_embeds_dispatch_size, vit.gbs, n, vit.dp)

    rl.actor_update_dispatch_size = rl.actor_update_dispatch_size or train_gbs * n // actor.dp
    _check_divides("Actor Update", train_gbs, n, rl.actor_update_dispatch_size)

    # -- algorithm-specific -----------------------------------------------------------------------
    _require(len(rl.verifier_function) == len(rl.verifier_weight),
             "verifier_function and verifier_weight must have the same length")
    max_tokens = gen.sampling_config["max_tokens"]
    if rl.overlong_buffer_enable:
        _require(rl.overlong_buffer < max_tokens,
                 f"overlong_buffer {rl.overlong_buffer} must be < max_tokens {max_tokens}")
        _require(rl.rollout_max_tokens == max_tokens,
                 f"rollout_max_tokens {rl.rollout_max_tokens} must equal max_tokens {max_tokens}")
    if rl.clip_higher_enable:
        _require(rl.clip_ratio_low <= rl.clip_ratio_high,
                 "clip_ratio_low must be <= clip_ratio_high")
    if rl.filter_groups_enable:
        _require(rl.filter_groups_metric in rl.verifier_function,
                 f"filter_groups_metric '{rl.filter_groups_metric}' must be one of the "
                 f"verifier functions {rl.verifier_function}")
        rl.filter_groups_metric += "_rewards/mean"
    _require(not (rl.partial_rollout_max_split > 1 and rl.guarantee_order),
             "partial rollout cannot be combined with guarantee_order")
    _require(not (rl.partial_rollout_max_split > 1 and rl.multi_turn_enable),
             "partial rollout cannot be combined with the multi-turn tool loop")
    _require(not (rl.partial_rollout_max_split > 1 and (actor_config.stage or "") == "ray_ppo"),
             "partial rollout is served by the GRPO and DAPO trainers only")
    if rl.multi_turn_enable:
        _require(rl.max_total_response_length >= max_tokens,
                 "max_total_response_length must be >= sampling max_tokens in multi-turn mode")
        _require(rl.async_engine, "multi-turn rollout needs async_engine=true")


_PROMPT_TYPE_HANDLERS = (
    "AlpacaStyleInstructionHandler", "AlpacaStylePairwiseHandler",
    "AlpacaStyleProcessRewardHandler", "R1AlpacaStyleInstructionHandler",
    "Math17kAlpacaStyleInstructionHandler",
)


def validate_data_handler_config(config) -> None:
    """Checks of ``cli/preprocess_data.py`` options (reference: validate_config.py:522-543)."""
    if config.prompt_type is not None and config.handler_name not in _PROMPT_TYPE_HANDLERS:
        raise ValueError(f"prompt_type needs a handler out of {list(_PROMPT_TYPE_HANDLERS)}")
    if config.merge_group_keys is not None and not os.path.isdir(config.input):
        raise ValueError(f"{config.input} is not a directory")
    out_dir = os.path.dirname(config.output_prefix)
    if not os.path.isdir(out_dir):
        raise ValueError(f"{out_dir} is not a directory")
    if config.neat_pack and not config.pack:
        raise ValueError("neat_pack requires pack")
    if config.enable_thinking and config.prompt_type != "qwen3":
        raise ValueError("enable_thinking is only available with the qwen3 prompt type")
