"""Zero-copy binding of training parameters as rollout weights.

When the rollout layout equals the training layout (same TP, PP = 1, no EP change) nothing has
to move: the rollout model runner can read the Megatron-layout tensors directly, because its
kernels address q/k/v heads through ``QKVLayout`` (interleaved or not) and ``linear_fc1`` is
already ``[gate; up]``.  This is the degenerate -- and fastest -- case of resharding; the
general case (TP shrink/grow, PP gather, EP re-homing) is handled by ``reshard.planner`` +
the reshard kernel.
"""
from __future__ import annotations

from ..models import lora
from ..models.gpt import GPTModel, MLP
from ..rollout.model_runner import LayerWeights, RolloutWeights


def alias_rollout_weights(model: GPTModel) -> RolloutWeights:
    layers = []
    for layer in model.decoder.layers:
        sa = layer.self_attention
        if getattr(layer.cfg, "multi_latent_attention", False):
            if not sa.rollout_supported():
                raise NotImplementedError(
                    "rollout of latent attention needs query/key and value heads of one common size 64 or 128 "
                    f"(got {sa.qd} / {sa.vd}): the paged KV cache stores full per-head keys and values")
            kw = dict(input_norm=layer.input_layernorm.weight.data, qkv_w=None, qkv_b=None, mla=sa,
                      o_w=sa.linear_proj.weight.data, post_norm=layer.pre_mlp_layernorm.weight.data)
        else:
            kw = _attention_weights(layer, sa)
        if isinstance(layer.mlp, MLP):
            kw.update(gate_up_w=lora.merged_weight(layer.mlp.linear_fc1),
                      down_w=lora.merged_weight(layer.mlp.linear_fc2))
        else:
            kw.update(moe=layer.mlp.rollout_view())
        layers.append(LayerWeights(**kw))
    first = model.decoder.layers[0].self_attention
    if getattr(model.cfg, "multi_latent_attention", False):
        from ..ops import QKVLayout

        layout = QKVLayout(first.nh, first.nh, first.qd, interleaved=True)
    else:
        layout = first.layout
    return RolloutWeights(
        embed=model.embedding.word_embeddings.weight.data,
        layers=layers,
        final_norm=model.decoder.final_layernorm.weight.data,
        lm_head=model.output_weight().data,
        qkv_layout=layout,
        vocab_start=model.vocab_start,
    )


def _attention_weights(layer, sa) -> dict:
    return dict(
        input_norm=layer.input_layernorm.weight.data,
        qkv_w=lora.merged_weight(sa.linear_qkv),       # W + (alpha/r) B A when adapted
        qkv_b=sa.linear_qkv.bias.data if sa.linear_qkv.bias is not None else None,
        o_w=lora.merged_weight(sa.linear_proj),
        post_norm=layer.pre_mlp_layernorm.weight.data,
        q_norm=sa.q_layernorm.weight.data if sa.q_layernorm is not None else None,
        k_norm=sa.k_layernorm.weight.data if sa.k_layernorm is not None else None,
    )
