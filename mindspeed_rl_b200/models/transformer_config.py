"""Architecture description consumed by the training model and the rollout model runner."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch


def parse_noop_layers(value) -> list:
    """``noop_layers`` as a list of slot indices (accepts a list or a comma-separated string)."""
    if value is None or value == "":
        return []
    if isinstance(value, str):
        return sorted({int(x) for x in value.split(",") if x.strip()})
    if isinstance(value, int):
        return [value]
    return sorted({int(x) for x in value})


@dataclass
class TransformerConfig:
    num_layers: int
    hidden_size: int
    ffn_hidden_size: int
    num_attention_heads: int
    num_query_groups: int
    vocab_size: int
    kv_channels: Optional[int] = None
    norm_epsilon: float = 1e-6
    rotary_base: float = 1_000_000.0
    max_position_embeddings: int = 32768
    add_qkv_bias: bool = False
    qk_layernorm: bool = False
    untie_embeddings_and_output_weights: bool = True
    init_method_std: float = 0.02
    # MoE
    num_experts: Optional[int] = None
    moe_router_topk: int = 2
    moe_ffn_hidden_size: Optional[int] = None
    n_shared_experts: Optional[int] = None
    norm_topk_prob: bool = False
    moe_router_score_function: str = "softmax"
    moe_aux_loss_coeff: float = 0.0
    first_k_dense_replace: int = 0
    moe_router_topk_scaling_factor: Optional[float] = None
    moe_router_enable_expert_bias: bool = False
    moe_router_num_groups: Optional[int] = None
    moe_router_group_topk: Optional[int] = None
    # multi-head latent attention (DeepSeek): low-rank query / key-value bottlenecks
    multi_latent_attention: bool = False
    q_lora_rank: Optional[int] = None
    kv_lora_rank: Optional[int] = None
    qk_head_dim: int = 128                # non-rotary part of a query / key head
    qk_pos_emb_head_dim: int = 64         # rotary part
    v_head_dim: int = 128
    # rope scaling (YaRN); None = plain RoPE
    rope_scaling: Optional[dict] = None
    # numerics / memory
    params_dtype: torch.dtype = torch.bfloat16
    recompute_granularity: Optional[str] = "full"   # "full" -> keep only layer inputs
    recompute_method: Optional[str] = None          # "block": only the first recompute_num_layers layers
    recompute_num_layers: Optional[int] = None
    recompute_activation_function: bool = False     # rebuild silu(g)*u in the backward instead of storing it
    moe_p2p_dispatch_rows: int = 0                  # rows of the peer-memory expert slabs (0: all-to-all collectives)
    moe_p2p_overflow_fallback: bool = True          # a routing that overflows a slab takes the all-to-all path for that call
    swap_attention: bool = False                    # kept activations wait for the backward in pinned host memory
    # which parts of a layer take part: input_norm, self_attention, post_attention_norm, mlp
    swap_modules: tuple = ("input_norm", "self_attention", "post_attention_norm", "mlp")
    # parallel sizes seen by the model code
    tensor_model_parallel_size: int = 1
    sequence_parallel: bool = False
    expert_model_parallel_size: int = 1
    # value/reward head
    value_head: bool = False
    # LoRA
    lora_r: int = 0
    lora_alpha: int = 16
    lora_target_modules: tuple = ()

    def __post_init__(self):
        if self.kv_channels is None:
            self.kv_channels = self.hidden_size // self.num_attention_heads
        if self.num_query_groups is None:
            self.num_query_groups = self.num_attention_heads
        if self.multi_latent_attention:
            if not self.kv_lora_rank:
                raise ValueError("multi_latent_attention needs kv_lora_rank")
            # the rollout engine stores full per-head keys (one KV head per query head)
            self.num_query_groups = self.num_attention_heads
            self.kv_channels = self.qk_head_dim + self.qk_pos_emb_head_dim

    @property
    def head_dim(self) -> int:
        return self.kv_channels

    @property
    def is_moe(self) -> bool:
        return bool(self.num_experts)

    def layer_is_moe(self, layer_idx: int) -> bool:
        return self.is_moe and layer_idx >= (self.first_k_dense_replace or 0)

    @classmethod
    def from_megatron(cls, cfg, **overrides) -> "TransformerConfig":
        """Build from a :class:`~mindspeed_rl_b200.config.MegatronConfig`."""
        nqg = cfg.num_query_groups if cfg.group_query_attention else cfg.num_attention_heads
        vocab = cfg.padded_vocab_size
        rope_scaling = None
        if getattr(cfg, "rope_scaling_type", None) == "yarn":
            rope_scaling = dict(
                factor=cfg.rope_scaling_factor,
                original_max_position_embeddings=(cfg.rope_scaling_original_max_position_embeddings
                                                  or cfg.original_max_position_embeddings or 4096),
                beta_fast=cfg.beta_fast, beta_slow=cfg.beta_slow, mscale=cfg.rope_scaling_mscale,
                mscale_all_dim=cfg.rope_scaling_mscale_all_dim)
        kw = dict(
            # the training config counts layer slots; empty (no-op) slots hold no layer
            num_layers=cfg.num_layers - len(parse_noop_layers(getattr(cfg, "noop_layers", None))),
            hidden_size=cfg.hidden_size,
            ffn_hidden_size=cfg.ffn_hidden_size, num_attention_heads=cfg.num_attention_heads,
            num_query_groups=nqg, vocab_size=vocab, kv_channels=cfg.kv_channels,
            norm_epsilon=cfg.norm_epsilon, rotary_base=float(cfg.rotary_base),
            max_position_embeddings=cfg.max_position_embeddings or 32768,
            add_qkv_bias=bool(cfg.add_qkv_bias), qk_layernorm=bool(cfg.qk_layernorm),
            untie_embeddings_and_output_weights=bool(cfg.untie_embeddings_and_output_weights),
            init_method_std=cfg.init_method_std, num_experts=cfg.num_experts,
            moe_router_topk=cfg.moe_router_topk, moe_ffn_hidden_size=cfg.moe_ffn_hidden_size,
            n_shared_experts=cfg.n_shared_experts, norm_topk_prob=bool(cfg.norm_topk_prob),
            moe_router_score_function=cfg.moe_router_score_function,
            moe_aux_loss_coeff=cfg.moe_aux_loss_coeff or 0.0,
            first_k_dense_replace=cfg.first_k_dense_replace or 0,
            moe_router_topk_scaling_factor=cfg.moe_router_topk_scaling_factor,
            moe_router_enable_expert_bias=bool(cfg.moe_router_enable_expert_bias),
            moe_router_num_groups=cfg.moe_router_num_groups,
            moe_router_group_topk=cfg.moe_router_group_topk,
            rope_scaling=rope_scaling,
            multi_latent_attention=bool(getattr(cfg, "multi_latent_attention", False)),
            q_lora_rank=getattr(cfg, "q_lora_rank", None), kv_lora_rank=getattr(cfg, "kv_lora_rank", None),
            qk_head_dim=getattr(cfg, "qk_head_dim", None) or 128,
            qk_pos_emb_head_dim=getattr(cfg, "qk_pos_emb_head_dim", None) or 64,
            v_head_dim=getattr(cfg, "v_head_dim", None) or 128,
            params_dtype=torch.bfloat16 if cfg.bf16 else torch.float32,
            recompute_granularity=cfg.recompute_granularity, recompute_method=cfg.recompute_method,
            recompute_num_layers=cfg.recompute_num_layers,
            recompute_activation_function=bool(cfg.recompute_activation_function),
            swap_attention=bool(getattr(cfg, "swap_attention", False)),
            swap_modules=_name_tuple(getattr(cfg, "swap_modules", None)
                                     or "input_norm,self_attention,post_attention_norm"),
            tensor_model_parallel_size=cfg.tensor_model_parallel_size,
            sequence_parallel=bool(cfg.sequence_parallel) and cfg.tensor_model_parallel_size > 1,
            expert_model_parallel_size=cfg.expert_model_parallel_size,
            lora_r=cfg.lora_r if cfg.lora_target_modules else 0, lora_alpha=cfg.lora_alpha,
            lora_target_modules=tuple(cfg.lora_target_modules or ()),
        )
        kw.update(overrides)
        return cls(**kw)


def _name_tuple(v) -> tuple:
    """``"a, b"`` or a sequence of names -> tuple of stripped names."""
    if isinstance(v, str):
        v = v.split(",")
    return tuple(str(x).strip() for x in v if str(x).strip())
