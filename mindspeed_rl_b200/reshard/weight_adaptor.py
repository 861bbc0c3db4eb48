"""Name mapping between rollout-side (Hugging Face / vLLM style) and training-side (Megatron-core
style) parameters, per architecture, plus the layer bookkeeping of pipeline stages.

The rollout engine of this repository consumes training tensors directly (``reshard/alias.py``,
``reshard/planner.py``), so nothing here moves data.  The registry exists for what still talks in
rollout-side names: checkpoint conversion, external inference engines fed from a training job,
debugging dumps.  A mapping is a table of ``(rollout pattern, training pattern)`` pairs with
``{i}`` for the layer number and ``{e}`` for an expert; fused tensors (``qkv_proj``, ``gate_up_proj``)
map to the single fused training tensor.

Reference: ``mindspeed_rl/workers/resharding/weight_adaptor.py:50-730`` (``MegatronVLLMWeightAdaptor``
and its per-architecture subclasses, ``get_weight_adaptor``).
"""
from __future__ import annotations

import re
from typing import Dict, List, Optional, Sequence, Tuple

_DENSE = [
    ("model.embed_tokens.weight", "embedding.word_embeddings.weight"),
    ("model.norm.weight", "decoder.final_layernorm.weight"),
    ("lm_head.weight", "output_layer.weight"),
    ("model.layers.{i}.input_layernorm.weight", "decoder.layers.{i}.input_layernorm.weight"),
    ("model.layers.{i}.self_attn.qkv_proj.weight", "decoder.layers.{i}.self_attention.linear_qkv.weight"),
    ("model.layers.{i}.self_attn.qkv_proj.bias", "decoder.layers.{i}.self_attention.linear_qkv.bias"),
    ("model.layers.{i}.self_attn.o_proj.weight", "decoder.layers.{i}.self_attention.linear_proj.weight"),
    ("model.layers.{i}.post_attention_layernorm.weight", "decoder.layers.{i}.pre_mlp_layernorm.weight"),
    ("model.layers.{i}.mlp.gate_up_proj.weight", "decoder.layers.{i}.mlp.linear_fc1.weight"),
    ("model.layers.{i}.mlp.down_proj.weight", "decoder.layers.{i}.mlp.linear_fc2.weight"),
]
_QK_NORM = [
    ("model.layers.{i}.self_attn.q_norm.weight", "decoder.layers.{i}.self_attention.q_layernorm.weight"),
    ("model.layers.{i}.self_attn.k_norm.weight", "decoder.layers.{i}.self_attention.k_layernorm.weight"),
]
_MOE = [
    ("model.layers.{i}.mlp.gate.weight", "decoder.layers.{i}.mlp.router.weight"),
    ("model.layers.{i}.mlp.experts.w13_weight", "decoder.layers.{i}.mlp.experts.weight1"),
    ("model.layers.{i}.mlp.experts.w2_weight", "decoder.layers.{i}.mlp.experts.weight2"),
    ("model.layers.{i}.mlp.shared_experts.gate_up_proj.weight", "decoder.layers.{i}.mlp.shared_experts.linear_fc1.weight"),
    ("model.layers.{i}.mlp.shared_experts.down_proj.weight", "decoder.layers.{i}.mlp.shared_experts.linear_fc2.weight"),
]
_MLA = [
    ("model.layers.{i}.self_attn.q_a_proj.weight", "decoder.layers.{i}.self_attention.linear_q_down_proj.weight"),
    ("model.layers.{i}.self_attn.q_a_layernorm.weight", "decoder.layers.{i}.self_attention.q_layernorm.weight"),
    ("model.layers.{i}.self_attn.q_b_proj.weight", "decoder.layers.{i}.self_attention.linear_q_up_proj.weight"),
    ("model.layers.{i}.self_attn.kv_a_proj_with_mqa.weight", "decoder.layers.{i}.self_attention.linear_kv_down_proj.weight"),
    ("model.layers.{i}.self_attn.kv_a_layernorm.weight", "decoder.layers.{i}.self_attention.kv_layernorm.weight"),
    ("model.layers.{i}.self_attn.kv_b_proj.weight", "decoder.layers.{i}.self_attention.linear_kv_up_proj.weight"),
    ("model.layers.{i}.mlp.gate.e_score_correction_bias", "decoder.layers.{i}.mlp.router.expert_bias"),
]


_VISION = [      # Qwen2.5-VL: vision tower ("visual.") beside the language model
    ("visual.patch_embed.proj.weight", "vision_model.patch_embed.weight"),
    ("visual.blocks.{i}.norm1.weight", "vision_model.blocks.{i}.norm1.weight"),
    ("visual.blocks.{i}.norm2.weight", "vision_model.blocks.{i}.norm2.weight"),
    ("visual.blocks.{i}.attn.qkv.weight", "vision_model.blocks.{i}.qkv.weight"),
    ("visual.blocks.{i}.attn.qkv.bias", "vision_model.blocks.{i}.qkv.bias"),
    ("visual.blocks.{i}.attn.proj.weight", "vision_model.blocks.{i}.proj.weight"),
    ("visual.blocks.{i}.attn.proj.bias", "vision_model.blocks.{i}.proj.bias"),
    ("visual.blocks.{i}.mlp.gate_up_proj.weight", "vision_model.blocks.{i}.gate_up.weight"),
    ("visual.blocks.{i}.mlp.gate_up_proj.bias", "vision_model.blocks.{i}.gate_up.bias"),
    ("visual.blocks.{i}.mlp.down_proj.weight", "vision_model.blocks.{i}.down.weight"),
    ("visual.blocks.{i}.mlp.down_proj.bias", "vision_model.blocks.{i}.down.bias"),
    ("visual.merger.ln_q.weight", "vision_model.merger_norm.weight"),
    ("visual.merger.mlp.0.weight", "vision_model.merger.0.weight"),
    ("visual.merger.mlp.0.bias", "vision_model.merger.0.bias"),
    ("visual.merger.mlp.2.weight", "vision_model.merger.2.weight"),
    ("visual.merger.mlp.2.bias", "vision_model.merger.2.bias"),
]


def _compile(pattern: str) -> re.Pattern:
    rx = re.escape(pattern).replace(r"\{i\}", r"(?P<i>\d+)").replace(r"\{e\}", r"(?P<e>\d+)")
    return re.compile("^" + rx + "$")


class WeightAdaptor:
    """Table-driven name mapper of one architecture."""

    def __init__(self, arch: str, table: Sequence[Tuple[str, str]]):
        self.arch = arch
        self.table = list(table)
        self._i2t = [(_compile(a), b) for a, b in self.table]
        self._t2i = [(_compile(b), a) for a, b in self.table]

    @staticmethod
    def _apply(rules, name: str) -> Optional[str]:
        for rx, target in rules:
            m = rx.match(name)
            if m:
                return target.format(**{k: v for k, v in m.groupdict().items() if v is not None})
        return None

    def replace_name_i2t(self, inference_name: str) -> str:
        """Rollout-side name -> training-side name (``KeyError`` when the table has no such tensor)."""
        out = self._apply(self._i2t, inference_name)
        if out is None:
            raise KeyError(f"{self.arch}: no training-side tensor for {inference_name!r}")
        return out

    def replace_name_t2i(self, training_name: str) -> str:
        out = self._apply(self._t2i, training_name)
        if out is None:
            raise KeyError(f"{self.arch}: no rollout-side tensor for {training_name!r}")
        return out

    def convert_weight_name_meta(self, weight_names: Sequence[str]) -> List[str]:
        """Rollout-side names that exist on the training side, in the given order (tensors without a
        counterpart, e.g. rotary caches, are dropped)."""
        return [n for n in weight_names if self._apply(self._i2t, n) is not None]

    # ---- pipeline bookkeeping ------------------------------------------------------------------------
    @staticmethod
    def layer_of(name: str) -> Optional[int]:
        m = re.search(r"(?:^|\.)layers\.(\d+)\.", name)
        return int(m.group(1)) if m else None

    @staticmethod
    def global2local_layer(name: str, num_layer_list: Sequence[int], noop_layers: Sequence[int] = ()
                           ) -> Tuple[int, str]:
        """``(pipeline stage, name with the stage-local layer number)`` of a layer tensor.
        ``num_layer_list[s]`` counts the layer slots of stage ``s`` including no-op slots; real layers
        are numbered without the no-op slots on the rollout side."""
        g = WeightAdaptor.layer_of(name)
        if g is None:
            raise ValueError(f"{name!r} does not belong to a layer")
        real = [i for i in range(sum(num_layer_list)) if i not in set(noop_layers)]
        if g >= len(real):
            raise ValueError(f"layer {g} is outside the model ({len(real)} layers)")
        slot = real[g]
        start = 0
        for stage, n in enumerate(num_layer_list):
            if slot < start + n:
                local = slot - start
                return stage, re.sub(r"layers\.\d+\.", f"layers.{local}.", name, count=1)
            start += n
        raise ValueError(f"layer {g} is outside the model")

    def get_weight_names_per_pp(self, num_layer_list: Sequence[int], names: Sequence[str],
                                noop_layers: Sequence[int] = ()) -> List[List[str]]:
        """Rollout-side names held by every pipeline stage: layer tensors by the stage of their layer,
        the embedding on the first stage, final norm and head on the last."""
        out: List[List[str]] = [[] for _ in num_layer_list]
        for n in names:
            if self.layer_of(n) is not None:
                stage, _ = self.global2local_layer(n, num_layer_list, noop_layers)
                out[stage].append(n)
            elif "embed_tokens" in n:
                out[0].append(n)
            else:
                out[-1].append(n)
        return out


_REGISTRY: Dict[str, WeightAdaptor] = {}


def register_weight_adaptor(archs: Sequence[str], table: Sequence[Tuple[str, str]]) -> None:
    for a in archs:
        _REGISTRY[a] = WeightAdaptor(a, table)


def get_weight_adaptor(arch: str) -> WeightAdaptor:
    if arch not in _REGISTRY:
        raise ValueError(f"no weight adaptor for architecture {arch!r}; known: {sorted(_REGISTRY)}")
    return _REGISTRY[arch]


register_weight_adaptor(["Qwen2ForCausalLM", "LlamaForCausalLM", "CustomQwen2ForCausalLM"], _DENSE)
register_weight_adaptor(["Qwen3ForCausalLM"], _DENSE + _QK_NORM)
register_weight_adaptor(["Qwen2_5_VLForConditionalGeneration", "Qwen2VLForConditionalGeneration"], _DENSE + _VISION)
register_weight_adaptor(["Qwen3MoeForCausalLM", "CustomQwen3MoeForCausalLM"], _DENSE + _QK_NORM + _MOE)
register_weight_adaptor(["DeepseekV2ForCausalLM", "DeepseekV3ForCausalLM", "CustomDeepseekV3ForCausalLM"],
                        [r for r in _DENSE if "qkv_proj" not in r[0]] + _MLA + _MOE)
