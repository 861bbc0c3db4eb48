"""Hugging Face <-> mcore checkpoint conversion for the supported decoder families
(Qwen2 / Qwen2.5 / Qwen3 dense, Qwen3-MoE).

HF keeps ``q_proj / k_proj / v_proj``, ``gate_proj / up_proj`` and one tensor per expert; mcore
keeps the fused, sharded layouts the training backend computes with:

* ``linear_qkv``: per TP shard, per KV group ``[q_0 .. q_{rep-1}, k, v]`` rows (interleaved);
* ``linear_fc1``: per TP shard ``[gate_shard; up_shard]``;
* ``linear_proj`` / ``linear_fc2``: column-sharded (input dim);
* embeddings / LM head: row-sharded over the vocabulary;
* MoE (``moe_grouped_gemm``): ``experts.weight1 [H, E_local * 2 * F_e]`` (per expert ``[gate | up]``
  columns) and ``experts.weight2 [E_local * F_e, H]``; experts are spread over ``ep`` ranks
  (``tp * ep`` with ``moe_tp_extend_ep``).

The HF key map mirrors ``configs/checkpoint/model_cfg.json`` of the reference (q/k/v/o_proj,
gate/up/down_proj, norms, ``score`` for reward models); the external converter the reference
relies on (MindSpeed-LLM ``checkpoint_convert``) does not exist here, hence this module.
"""
from __future__ import annotations

import glob
import json
import os
from types import SimpleNamespace
from typing import Dict, List, Optional

import torch

from .mcore import CHECKPOINT_VERSION, TRACKER, checkpoint_dir, rank_dir_name, read_tracker


# ----------------------------------------------------------------------------------------------
# HF side I/O
# ----------------------------------------------------------------------------------------------
def load_hf_state(path: str) -> Dict[str, torch.Tensor]:
    files = sorted(glob.glob(os.path.join(path, "*.safetensors")))
    state: Dict[str, torch.Tensor] = {}
    if files:
        from safetensors.torch import load_file

        for f in files:
            state.update(load_file(f))
        return state
    for f in sorted(glob.glob(os.path.join(path, "pytorch_model*.bin"))):
        state.update(torch.load(f, map_location="cpu", weights_only=True))
    if not state:
        raise FileNotFoundError(f"no safetensors / bin weights under {path}")
    return state


def save_hf_state(state: Dict[str, torch.Tensor], path: str, shard_bytes: int = 5 << 30) -> None:
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    shards, cur, size = [], {}, 0
    for k, v in state.items():
        n = v.numel() * v.element_size()
        if cur and size + n > shard_bytes:
            shards.append(cur)
            cur, size = {}, 0
        cur[k] = v.contiguous()
        size += n
    shards.append(cur)
    index = {"metadata": {"total_size": sum(v.numel() * v.element_size() for v in state.values())},
             "weight_map": {}}
    for i, sh in enumerate(shards):
        name = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        save_file(sh, os.path.join(path, name), metadata={"format": "pt"})
        for k in sh:
            index["weight_map"][k] = name
    with open(os.path.join(path, "model.safetensors.index.json"), "w") as fh:
        json.dump(index, fh, indent=1)


# ----------------------------------------------------------------------------------------------
# layout transforms (whole-model tensors, no sharding)
# ----------------------------------------------------------------------------------------------
def qkv_hf_to_mcore(q, k, v, nh: int, nkv: int, hd: int) -> torch.Tensor:
    """[nh*hd, H], [nkv*hd, H], [nkv*hd, H] -> interleaved [(nh+2nkv)*hd, H] (also biases)."""
    rep = nh // nkv
    tail = q.shape[1:]
    g = torch.cat([q.reshape(nkv, rep * hd, *tail), k.reshape(nkv, hd, *tail), v.reshape(nkv, hd, *tail)], dim=1)
    return g.reshape((nh + 2 * nkv) * hd, *tail)


def qkv_mcore_to_hf(qkv, nh: int, nkv: int, hd: int):
    rep = nh // nkv
    tail = qkv.shape[1:]
    g = qkv.reshape(nkv, (rep + 2) * hd, *tail)
    q = g[:, :rep * hd].reshape(nh * hd, *tail)
    k = g[:, rep * hd:(rep + 1) * hd].reshape(nkv * hd, *tail)
    v = g[:, (rep + 1) * hd:].reshape(nkv * hd, *tail)
    return q, k, v


def shard_rows(t: torch.Tensor, tp: int, r: int) -> torch.Tensor:
    return t.chunk(tp, dim=0)[r].contiguous()


def shard_cols(t: torch.Tensor, tp: int, r: int) -> torch.Tensor:
    return t.chunk(tp, dim=1)[r].contiguous()


def shard_qkv(qkv_full: torch.Tensor, nkv: int, tp: int, r: int) -> torch.Tensor:
    """Interleaved QKV is sharded by KV groups."""
    g = qkv_full.reshape(nkv, -1, *qkv_full.shape[1:])
    part = g.chunk(tp, dim=0)[r]
    return part.reshape(-1, *qkv_full.shape[1:]).contiguous()


def shard_fc1(gate: torch.Tensor, up: torch.Tensor, tp: int, r: int) -> torch.Tensor:
    return torch.cat([gate.chunk(tp, 0)[r], up.chunk(tp, 0)[r]], dim=0).contiguous()


def _layer_split(num_layers: int, pp: int, num_layer_list: Optional[List[int]] = None) -> List[List[int]]:
    sizes = list(num_layer_list) if num_layer_list else [num_layers // pp] * pp
    if sum(sizes) != num_layers:
        raise ValueError(f"layer split {sizes} does not sum to {num_layers}")
    out, s = [], 0
    for n in sizes:
        out.append(list(range(s, s + n)))
        s += n
    return out


# ---- multi-head latent attention (DeepSeek) ---------------------------------------------------
# Hugging Face stores the rotary slice of a head with (even, odd) pairs interleaved; the kernels here
# rotate halves, so the rotary rows are reordered on the way in and back on the way out.  The tensor
# names come from the architecture's name table (``reshard.weight_adaptor``).
def _rope_perm(d: int, inverse: bool = False) -> torch.Tensor:
    perm = torch.cat([torch.arange(0, d, 2), torch.arange(1, d, 2)])
    return torch.argsort(perm) if inverse else perm


def _mla_reorder(name: str, w: torch.Tensor, cfg, inverse: bool) -> torch.Tensor:
    nope, rope = cfg.qk_head_dim, cfg.qk_pos_emb_head_dim
    perm = _rope_perm(rope, inverse)
    if name.endswith(("q_b_proj.weight", "q_proj.weight")):
        v = w.view(-1, nope + rope, w.shape[-1]).clone()          # [heads, nope + rope, in]
        v[:, nope:] = v[:, nope:][:, perm]
        return v.reshape(w.shape)
    if name.endswith("kv_a_proj_with_mqa.weight"):
        out = w.clone()
        out[cfg.kv_lora_rank:] = w[cfg.kv_lora_rank:][perm]
        return out
    return w


_MLA_HF = ("q_a_proj.weight", "q_a_layernorm.weight", "q_b_proj.weight", "kv_a_proj_with_mqa.weight",
           "kv_a_layernorm.weight", "kv_b_proj.weight")


def _mla_hf_to_mcore(hf, sd, src: str, dst: str, layer: int, local: int, cfg, tp: int, t: int) -> None:
    from ..reshard.weight_adaptor import get_weight_adaptor

    ad = get_weight_adaptor("DeepseekV3ForCausalLM")
    for tail in _MLA_HF:
        name = src + "self_attn." + tail
        if name not in hf:
            continue
        target = ad.replace_name_i2t(name).replace(f"layers.{layer}.", f"layers.{local}.", 1)
        w = _mla_reorder(name, hf[name], cfg, inverse=False)
        sd[target] = shard_rows(w, tp, t) if tail in ("q_b_proj.weight", "kv_b_proj.weight") else w.clone()
    if src + "self_attn.q_proj.weight" in hf:       # no query bottleneck (DeepSeek-V2-Lite)
        w = _mla_reorder(src + "self_attn.q_proj.weight", hf[src + "self_attn.q_proj.weight"], cfg, inverse=False)
        sd[dst + "self_attention.linear_q_proj.weight"] = shard_rows(w, tp, t)
    sd[dst + "self_attention.linear_proj.weight"] = shard_cols(hf[src + "self_attn.o_proj.weight"], tp, t)


def _mla_mcore_to_hf(shards, hf, src: str, dst: str, layer: int, local: int, p: int, cfg, tp: int) -> None:
    from ..reshard.weight_adaptor import get_weight_adaptor

    ad = get_weight_adaptor("DeepseekV3ForCausalLM")
    s0 = shards[(0, p, 0)]
    for key in list(s0):
        if not key.startswith(src + "self_attention.") or key.endswith("linear_proj.weight"):
            continue
        if key.endswith("linear_q_proj.weight"):
            name = dst + "self_attn.q_proj.weight"
        else:
            name = ad.replace_name_t2i(key.replace(f"layers.{local}.", f"layers.{layer}.", 1))
        split = key.endswith(("linear_q_up_proj.weight", "linear_kv_up_proj.weight", "linear_q_proj.weight"))
        w = torch.cat([shards[(t, p, 0)][key] for t in range(tp)], 0) if split else s0[key]
        hf[name] = _mla_reorder(name, w, cfg, inverse=True).contiguous()
    hf[dst + "self_attn.o_proj.weight"] = torch.cat(
        [shards[(t, p, 0)][src + "self_attention.linear_proj.weight"] for t in range(tp)], 1)


# ----------------------------------------------------------------------------------------------
# HF -> mcore
# ----------------------------------------------------------------------------------------------
def hf_to_mcore(hf: Dict[str, torch.Tensor], cfg, tp: int = 1, pp: int = 1, ep: int = 1,
                moe_tp_extend_ep: bool = False, num_layer_list: Optional[List[int]] = None,
                orm: bool = False) -> Dict[tuple, Dict[str, torch.Tensor]]:
    """Returns ``{(tp_rank, pp_rank, ep_rank): state_dict}`` of mcore-named tensors.

    ``cfg`` needs ``num_layers, num_attention_heads, num_query_groups, head_dim (kv_channels),
    qk_layernorm, num_experts, untie_embeddings_and_output_weights``.
    """
    nh, nkv = cfg.num_attention_heads, cfg.num_query_groups
    hd = cfg.kv_channels or cfg.hidden_size // nh
    stages = _layer_split(cfg.num_layers, pp, num_layer_list)
    n_exp = cfg.num_experts or 0
    ep_total = ep * tp if (moe_tp_extend_ep and n_exp) else ep
    out: Dict[tuple, Dict[str, torch.Tensor]] = {}
    for t in range(tp):
        for p in range(pp):
            for e in range(ep):
                sd: Dict[str, torch.Tensor] = {}
                if p == 0:
                    sd["embedding.word_embeddings.weight"] = shard_rows(hf["model.embed_tokens.weight"], tp, t)
                for local, layer in enumerate(stages[p]):
                    src, dst = f"model.layers.{layer}.", f"decoder.layers.{local}."
                    sd[dst + "input_layernorm.weight"] = hf[src + "input_layernorm.weight"].clone()
                    sd[dst + "pre_mlp_layernorm.weight"] = hf[src + "post_attention_layernorm.weight"].clone()
                    mla = src + "self_attn.kv_a_proj_with_mqa.weight" in hf
                    if mla:
                        _mla_hf_to_mcore(hf, sd, src, dst, layer, local, cfg, tp, t)
                    else:
                        qkv = qkv_hf_to_mcore(hf[src + "self_attn.q_proj.weight"], hf[src + "self_attn.k_proj.weight"],
                                              hf[src + "self_attn.v_proj.weight"], nh, nkv, hd)
                        sd[dst + "self_attention.linear_qkv.weight"] = shard_qkv(qkv, nkv, tp, t)
                        if src + "self_attn.q_proj.bias" in hf:
                            qb = qkv_hf_to_mcore(hf[src + "self_attn.q_proj.bias"], hf[src + "self_attn.k_proj.bias"],
                                                 hf[src + "self_attn.v_proj.bias"], nh, nkv, hd)
                            sd[dst + "self_attention.linear_qkv.bias"] = shard_qkv(qb, nkv, tp, t)
                        sd[dst + "self_attention.linear_proj.weight"] = shard_cols(hf[src + "self_attn.o_proj.weight"], tp, t)
                    if src + "self_attn.q_norm.weight" in hf:
                        sd[dst + "self_attention.q_layernorm.weight"] = hf[src + "self_attn.q_norm.weight"].clone()
                        sd[dst + "self_attention.k_layernorm.weight"] = hf[src + "self_attn.k_norm.weight"].clone()
                    if src + "mlp.gate.weight" in hf:      # MoE layer
                        sd[dst + "mlp.router.weight"] = hf[src + "mlp.gate.weight"].clone()
                        if src + "mlp.gate.e_score_correction_bias" in hf:
                            sd[dst + "mlp.router.expert_bias"] = hf[src + "mlp.gate.e_score_correction_bias"].float().clone()
                        ep_rank = (e * tp + t) if moe_tp_extend_ep else e
                        per = n_exp // ep_total
                        w1, w2 = [], []
                        for x in range(ep_rank * per, (ep_rank + 1) * per):
                            g = hf[src + f"mlp.experts.{x}.gate_proj.weight"]
                            u = hf[src + f"mlp.experts.{x}.up_proj.weight"]
                            w1.append(torch.cat([g, u], dim=0).t())          # [H, 2F]
                            w2.append(hf[src + f"mlp.experts.{x}.down_proj.weight"].t())   # [F, H]
                        sd[dst + "mlp.experts.weight1"] = torch.cat(w1, dim=1).contiguous()
                        sd[dst + "mlp.experts.weight2"] = torch.cat(w2, dim=0).contiguous()
                        if src + "mlp.shared_expert.gate_proj.weight" in hf:
                            sd[dst + "mlp.shared_experts.linear_fc1.weight"] = shard_fc1(
                                hf[src + "mlp.shared_expert.gate_proj.weight"],
                                hf[src + "mlp.shared_expert.up_proj.weight"], tp, t)
                            sd[dst + "mlp.shared_experts.linear_fc2.weight"] = shard_cols(
                                hf[src + "mlp.shared_expert.down_proj.weight"], tp, t)
                    else:
                        sd[dst + "mlp.linear_fc1.weight"] = shard_fc1(hf[src + "mlp.gate_proj.weight"],
                                                                      hf[src + "mlp.up_proj.weight"], tp, t)
                        sd[dst + "mlp.linear_fc2.weight"] = shard_cols(hf[src + "mlp.down_proj.weight"], tp, t)
                if p == pp - 1:
                    sd["decoder.final_layernorm.weight"] = hf["model.norm.weight"].clone()
                    if orm and "score.weight" in hf:
                        sd["rm_head.weight"] = hf["score.weight"].float().clone()
                        sd["rm_head.bias"] = hf.get("score.bias", torch.zeros(hf["score.weight"].shape[0])).float()
                    if cfg.untie_embeddings_and_output_weights or pp > 1:
                        head = hf.get("lm_head.weight", hf["model.embed_tokens.weight"])
                        sd["output_layer.weight"] = shard_rows(head, tp, t)
                out[(t, p, e)] = sd
    return out


def write_mcore(shards: Dict[tuple, Dict[str, torch.Tensor]], root: str, tp: int, pp: int, ep: int,
                args: Optional[dict] = None, iteration: int = 0, release: bool = True) -> None:
    base = checkpoint_dir(root, iteration, release)
    for (t, p, e), sd in shards.items():
        d = os.path.join(base, rank_dir_name(t, p, pp, e, ep))
        os.makedirs(d, exist_ok=True)
        torch.save({"args": SimpleNamespace(**(args or {})), "checkpoint_version": CHECKPOINT_VERSION,
                    "iteration": iteration, "model": sd}, os.path.join(d, "model_optim_rng.pt"))
    with open(os.path.join(root, TRACKER), "w") as fh:
        fh.write("release" if release else str(iteration))


# ----------------------------------------------------------------------------------------------
# mcore -> HF
# ----------------------------------------------------------------------------------------------
def read_mcore(root: str, tp: int, pp: int, ep: int = 1) -> Dict[tuple, Dict[str, torch.Tensor]]:
    it, release = read_tracker(root)
    if it is None:
        raise FileNotFoundError(f"no {TRACKER} under {root}")
    base = checkpoint_dir(root, it, release)
    out = {}
    for t in range(tp):
        for p in range(pp):
            for e in range(ep):
                f = os.path.join(base, rank_dir_name(t, p, pp, e, ep), "model_optim_rng.pt")
                out[(t, p, e)] = torch.load(f, map_location="cpu", weights_only=False)["model"]
    return out


def mcore_to_hf(shards: Dict[tuple, Dict[str, torch.Tensor]], cfg, tp: int = 1, pp: int = 1, ep: int = 1,
                moe_tp_extend_ep: bool = False, num_layer_list: Optional[List[int]] = None
                ) -> Dict[str, torch.Tensor]:
    nh, nkv = cfg.num_attention_heads, cfg.num_query_groups
    hd = cfg.kv_channels or cfg.hidden_size // nh
    stages = _layer_split(cfg.num_layers, pp, num_layer_list)
    n_exp = cfg.num_experts or 0
    ep_total = ep * tp if (moe_tp_extend_ep and n_exp) else ep
    hf: Dict[str, torch.Tensor] = {}

    def cat(key, p, dim, e=0):
        return torch.cat([shards[(t, p, e)][key] for t in range(tp)], dim=dim)

    hf["model.embed_tokens.weight"] = cat("embedding.word_embeddings.weight", 0, 0)
    for p in range(pp):
        for local, layer in enumerate(stages[p]):
            src, dst = f"decoder.layers.{local}.", f"model.layers.{layer}."
            s0 = shards[(0, p, 0)]
            hf[dst + "input_layernorm.weight"] = s0[src + "input_layernorm.weight"]
            hf[dst + "post_attention_layernorm.weight"] = s0[src + "pre_mlp_layernorm.weight"]
            if src + "self_attention.linear_kv_down_proj.weight" in s0:
                _mla_mcore_to_hf(shards, hf, src, dst, layer, local, p, cfg, tp)
            else:
                q, k, v = qkv_mcore_to_hf(cat(src + "self_attention.linear_qkv.weight", p, 0), nh, nkv, hd)
                hf[dst + "self_attn.q_proj.weight"], hf[dst + "self_attn.k_proj.weight"], \
                    hf[dst + "self_attn.v_proj.weight"] = q.contiguous(), k.contiguous(), v.contiguous()
                if src + "self_attention.linear_qkv.bias" in s0:
                    qb, kb, vb = qkv_mcore_to_hf(cat(src + "self_attention.linear_qkv.bias", p, 0), nh, nkv, hd)
                    hf[dst + "self_attn.q_proj.bias"], hf[dst + "self_attn.k_proj.bias"], \
                        hf[dst + "self_attn.v_proj.bias"] = qb.contiguous(), kb.contiguous(), vb.contiguous()
                hf[dst + "self_attn.o_proj.weight"] = cat(src + "self_attention.linear_proj.weight", p, 1)
            if src + "self_attention.q_layernorm.weight" in s0 and src + "self_attention.k_layernorm.weight" in s0:
                hf[dst + "self_attn.q_norm.weight"] = s0[src + "self_attention.q_layernorm.weight"]
                hf[dst + "self_attn.k_norm.weight"] = s0[src + "self_attention.k_layernorm.weight"]
            if src + "mlp.router.weight" in s0:
                hf[dst + "mlp.gate.weight"] = s0[src + "mlp.router.weight"]
                if src + "mlp.router.expert_bias" in s0:
                    hf[dst + "mlp.gate.e_score_correction_bias"] = s0[src + "mlp.router.expert_bias"]
                per = n_exp // ep_total
                f_e = cfg.moe_ffn_hidden_size
                for t in range(tp if moe_tp_extend_ep else 1):
                    for e in range(ep):
                        rank = (e * tp + t) if moe_tp_extend_ep else e
                        sd = shards[(t, p, e)]
                        w1 = sd[src + "mlp.experts.weight1"].reshape(-1, per, 2 * f_e)   # [H, E_l, 2F]
                        w2 = sd[src + "mlp.experts.weight2"].reshape(per, f_e, -1)       # [E_l, F, H]
                        for j in range(per):
                            x = rank * per + j
                            gu = w1[:, j].t()
                            hf[dst + f"mlp.experts.{x}.gate_proj.weight"] = gu[:f_e].contiguous()
                            hf[dst + f"mlp.experts.{x}.up_proj.weight"] = gu[f_e:].contiguous()
                            hf[dst + f"mlp.experts.{x}.down_proj.weight"] = w2[j].t().contiguous()
            else:
                fc1 = [shards[(t, p, 0)][src + "mlp.linear_fc1.weight"].chunk(2, 0) for t in range(tp)]
                hf[dst + "mlp.gate_proj.weight"] = torch.cat([g for g, _ in fc1], 0)
                hf[dst + "mlp.up_proj.weight"] = torch.cat([u for _, u in fc1], 0)
                hf[dst + "mlp.down_proj.weight"] = cat(src + "mlp.linear_fc2.weight", p, 1)
    last = pp - 1
    hf["model.norm.weight"] = shards[(0, last, 0)]["decoder.final_layernorm.weight"]
    if "output_layer.weight" in shards[(0, last, 0)]:
        hf["lm_head.weight"] = cat("output_layer.weight", last, 0)
    if "rm_head.weight" in shards[(0, last, 0)]:
        hf["score.weight"] = shards[(0, last, 0)]["rm_head.weight"]
    return hf
