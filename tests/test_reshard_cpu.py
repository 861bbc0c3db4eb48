"""Resharding plan: every rollout rank's weights equal a direct sharding of the full model."""
import pytest
import torch

from mindspeed_rl_b200.checkpoint import convert as C
from mindspeed_rl_b200.models.gpt import GPTModel
from mindspeed_rl_b200.models.transformer_config import TransformerConfig
from mindspeed_rl_b200.parallel.state import RankLayout
from mindspeed_rl_b200.reshard.planner import (Slot, build_plan, execute_plan_torch, intervals, stage_layers,
                                               weights_from_buffer)


def _cfg(**kw):
    base = dict(num_layers=4, hidden_size=64, ffn_hidden_size=128, num_attention_heads=8, num_query_groups=4,
                vocab_size=256, kv_channels=16, add_qkv_bias=True, untie_embeddings_and_output_weights=True,
                params_dtype=torch.float32)
    base.update(kw)
    return TransformerConfig(**base)


def _shard(full, cfg, tp, r):
    out = {}
    for k, v in full.items():
        if k.endswith(("linear_qkv.weight", "linear_qkv.bias")):
            out[k] = C.shard_qkv(v, cfg.num_query_groups, tp, r)
        elif k.endswith("linear_fc1.weight"):
            g, u = v.chunk(2, 0)
            out[k] = C.shard_fc1(g, u, tp, r)
        elif k.endswith(("linear_proj.weight", "linear_fc2.weight")):
            out[k] = C.shard_cols(v, tp, r)
        elif k.endswith(("word_embeddings.weight", "output_layer.weight")):
            out[k] = C.shard_rows(v, tp, r)
        elif k.endswith(("linear_q_up_proj.weight", "linear_kv_up_proj.weight", "linear_q_proj.weight")):
            out[k] = C.shard_rows(v, tp, r)          # latent attention: whole heads, head-major
        else:
            out[k] = v.clone()
    return out


def _stage_state(sharded, layers, first, last):
    """Global-index state dict -> local-index state dict of one pipeline stage."""
    out = {}
    for k, v in sharded.items():
        if k.startswith("decoder.layers."):
            idx = int(k.split(".")[2])
            if idx in layers:
                out[f"decoder.layers.{layers.index(idx)}." + k.split(".", 3)[3]] = v
        elif k.startswith("embedding."):
            if first:
                out[k] = v
        elif last:
            out[k] = v
    return out


def _flatten(state):
    slots, off, chunks = {}, 0, []
    for k, v in state.items():
        slots[k] = Slot(off, tuple(v.shape))
        chunks.append(v.reshape(-1))
        pad = (-v.numel()) % 64
        if pad:
            chunks.append(torch.zeros(pad))
        off += v.numel() + pad
    return slots, torch.cat(chunks).contiguous()


def test_intervals_cover_destination():
    for n_src, n_dst in [(4, 2), (2, 4), (4, 4), (1, 8), (8, 1), (4, 1)]:
        n = 64
        for j in range(n_dst):
            got = intervals(n, n_src, n_dst, j)
            assert sum(p[3] for p in got) == n // n_dst
            pos = 0
            for s, s0, d0, ln in got:
                assert d0 == pos and 0 <= s0 and s0 + ln <= n // n_src
                assert s * (n // n_src) + s0 == j * (n // n_dst) + d0
                pos += ln


@pytest.mark.parametrize("tp_t,pp_t,tp_i,world", [(4, 1, 2, 4), (2, 2, 1, 4), (2, 1, 4, 4), (2, 2, 2, 8),
                                                   (4, 2, 2, 8), (1, 2, 2, 4)])
def test_plan_matches_direct_sharding(tp_t, pp_t, tp_i, world):
    _check_plan(_cfg(), tp_t, pp_t, tp_i, world)


# train TP x PP -> rollout TP of the shipped recipes (32B GRPO 4x4 -> 2, 32B DAPO long context 8x2 -> 4,
# Qwen3-32B 8x2 -> 8, LoRA 4x4 -> 4, 235B 2x16 -> 4 scaled to 2x4 -> 4), one of them with uneven stages
@pytest.mark.parametrize("tp_t,pp_t,tp_i,world,layer_list", [(4, 4, 2, 16, None), (8, 2, 4, 16, None),
                                                              (8, 2, 8, 16, None), (4, 4, 4, 16, [1, 2, 1, 1]),
                                                              (2, 4, 4, 8, None)])
def test_plan_for_recipe_layouts(tp_t, pp_t, tp_i, world, layer_list):
    cfg = _cfg(num_attention_heads=16, num_query_groups=8, kv_channels=8,
               num_layers=sum(layer_list) if layer_list else 4)
    _check_plan(cfg, tp_t, pp_t, tp_i, world, layer_list)


def _check_plan(cfg, tp_t, pp_t, tp_i, world, layer_list=None):
    full = GPTModel(cfg, seed=3).state_dict()
    train = RankLayout(world, tp=tp_t, pp=pp_t)
    layers = stage_layers(cfg.num_layers, pp_t, layer_list)
    buffers, tables = {}, [None] * pp_t
    for r in range(world):
        c = train.coords(r)
        st = _stage_state(_shard(full, cfg, tp_t, c["tp"]), layers[c["pp"]], c["pp"] == 0, c["pp"] == pp_t - 1)
        slots, flat = _flatten(st)
        tables[c["pp"]] = slots
        buffers[r] = flat.view(torch.uint8)
    for r in range(world):
        plan = build_plan(cfg, train, tp_i, r, tables, layers, lambda rank: 0, esz=4)
        dst = torch.zeros(plan.nbytes, dtype=torch.uint8)
        execute_plan_torch(plan, buffers, dst)
        j = r % tp_i
        want = _shard(full, cfg, tp_i, j)
        assert set(plan.tensors) == set(want)
        for name, (off, shape) in plan.tensors.items():
            got = dst[off:off + want[name].numel() * 4].view(torch.float32).view(shape)
            assert torch.equal(got, want[name]), name
        # all sources stay inside the rank's own model replica
        mp = [m for g in train.groups("tp", "pp") if r in g for m in g]
        assert {d[0] for d in plan.desc} <= set(mp)
        w = weights_from_buffer(cfg, tp_i, j, plan, dst, torch.float32)
        assert w.layers[0].qkv_w.shape[0] == (cfg.num_attention_heads + 2 * cfg.num_query_groups) // tp_i * cfg.kv_channels
        assert w.vocab_start == j * cfg.vocab_size // tp_i


def _moe_cfg(**kw):
    return _cfg(num_layers=2, num_experts=8, moe_router_topk=2, moe_ffn_hidden_size=32, **kw)


def _expert_shard(full, cfg, ep, r):
    """State dict of training expert-parallel rank ``r`` of ``ep``: its block of every layer's experts."""
    h, f, e = cfg.hidden_size, cfg.moe_ffn_hidden_size, cfg.num_experts
    per = e // ep
    out = {}
    for k, v in full.items():
        if k.endswith("experts.weight1"):
            out[k] = v.view(h, e, 2 * f)[:, r * per:(r + 1) * per].reshape(h, -1).contiguous()
        elif k.endswith("experts.weight2"):
            out[k] = v.view(e, f, h)[r * per:(r + 1) * per].reshape(-1, h).contiguous()
        else:
            out[k] = v.clone()
    return out


@pytest.mark.parametrize("ep_t,pp_t,ep_i,redundant", [(2, 1, 4, 0), (4, 1, 1, 0), (2, 2, 4, 0), (2, 1, 2, 1), (1, 1, 4, 1)])
def test_plan_rehomes_experts(ep_t, pp_t, ep_i, redundant):
    """Expert growth (EP2 -> EP4), expert replication (EP4 -> every rank holds all), experts gathered from
    pipeline stages, and a placement map with one redundant expert slot per rollout rank: every rollout
    rank's expert tensors hold exactly the logical experts it is said to host, in slot order."""
    from mindspeed_rl_b200.reshard.planner import ExpertPlacement
    from mindspeed_rl_b200.rollout.eplb import expert_map_from_counts

    cfg = _moe_cfg()
    full = GPTModel(cfg, seed=5).state_dict()
    world = 4 * pp_t
    train = RankLayout(world, pp=pp_t, ep=ep_t)
    layers = stage_layers(cfg.num_layers, pp_t)
    h, f, e = cfg.hidden_size, cfg.moe_ffn_hidden_size, cfg.num_experts
    buffers, tables = {}, [None] * pp_t
    for r in range(world):
        c, ec = train.coords(r), train.expert_coords(r)
        st = _stage_state(_expert_shard(full, cfg, ep_t, ec["ep"]), layers[c["pp"]], c["pp"] == 0, c["pp"] == pp_t - 1)
        slots, flat = _flatten(st)
        tables[c["pp"]] = slots
        buffers[r] = flat.view(torch.uint8)
    emap = None
    if redundant:
        torch.manual_seed(1)
        emap = expert_map_from_counts(torch.randint(1, 100, (cfg.num_layers, e)), ep_i, redundant)
    infer = RankLayout(world, ep=ep_i)
    for r in range(world):
        ei = infer.expert_coords(r)["ep"]
        mine = train.expert_coords(r)

        def hosted(layer, ei=ei):
            if emap is not None:
                return emap["layer_list"][layer]["device_list"][ei]["device_expert"]
            per = e // ep_i
            return list(range(ei * per, (ei + 1) * per))

        def src_rank(ep_index, stage, mine=mine):
            stage_rank = mine["etp"] + train.expert_tp * (ep_index + train.ep_total * mine["edp"])
            return train.rank_of(tp=stage_rank % train.tp, cp=(stage_rank // train.tp) % train.cp,
                                 dp=stage_rank // (train.tp * train.cp), pp=stage)

        plan = build_plan(cfg, train, 1, r, tables, layers, lambda rank: 0, esz=4,
                          experts=ExpertPlacement(e // ep_t, hosted, src_rank))
        dst = torch.zeros(plan.nbytes, dtype=torch.uint8)
        execute_plan_torch(plan, buffers, dst)
        for layer in range(cfg.num_layers):
            ids = hosted(layer)
            assert len(ids) == (e + redundant * ep_i) // ep_i and len(set(ids)) == len(ids)
            for name, ref in (("weight1", full[f"decoder.layers.{layer}.mlp.experts.weight1"].view(h, e, 2 * f)[:, ids]),
                              ("weight2", full[f"decoder.layers.{layer}.mlp.experts.weight2"].view(e, f, h)[ids])):
                off, shape = plan.tensors[f"decoder.layers.{layer}.mlp.experts.{name}"]
                got = dst[off:off + ref.numel() * 4].view(torch.float32).view(shape)
                assert torch.equal(got, ref.reshape(shape)), (r, layer, name)
            off, shape = plan.tensors[f"decoder.layers.{layer}.mlp.router.weight"]
            assert torch.equal(dst[off:off + e * h * 4].view(torch.float32).view(shape),
                               full[f"decoder.layers.{layer}.mlp.router.weight"])
        # expert sources are ranks of my own expert-data-parallel replica that own the shard
        for i, d in enumerate(plan.desc):
            assert train.expert_coords(d[0])["edp"] == mine["edp"] or plan.buf_of(i) == 0


def test_plan_carries_adapters_and_rollout_folds_them():
    """LoRA under a TP change (train TP2 -> rollout TP1 and TP4): ``B`` is cut like the weight's output rows,
    ``A`` like its input columns, and the rollout copy of the weight becomes ``W + (alpha / r) B A``."""
    from mindspeed_rl_b200.models import lora

    cfg = _cfg(num_layers=2, lora_r=4, lora_alpha=8, lora_target_modules=["linear_qkv", "linear_proj", "linear_fc1", "linear_fc2"])
    model = GPTModel(cfg, seed=7)
    torch.manual_seed(0)
    for hld in lora.holders(model):
        hld.lora_B.data.normal_(0, 0.05)                   # B starts at zero: make the fold visible
    full = model.state_dict()
    merged = {n: lora.merged_weight(m) for n, m in model.named_modules() if getattr(m, "lora_A", None) is not None}

    def shard_adapters(state, tp, r):
        out = _shard({k: v for k, v in state.items() if "lora_" not in k}, cfg, tp, r)
        for k, v in state.items():
            if k.endswith("linear_qkv.lora_B"):
                out[k] = C.shard_qkv(v, cfg.num_query_groups, tp, r)
            elif k.endswith("linear_fc1.lora_B"):
                g, u = v.chunk(2, 0)
                out[k] = C.shard_fc1(g, u, tp, r)
            elif k.endswith(("linear_proj.lora_A", "linear_fc2.lora_A")):
                out[k] = C.shard_cols(v, tp, r)
            elif "lora_" in k:
                out[k] = v.clone()
        return out

    tp_t = 2
    train = RankLayout(tp_t, tp=tp_t)
    layers = stage_layers(cfg.num_layers, 1)
    buffers, tables = {}, [None]
    for r in range(tp_t):
        slots, flat = _flatten(shard_adapters(full, tp_t, r))
        tables[0] = slots
        buffers[r] = flat.view(torch.uint8)
    for tp_i in (1, 2):
        world = max(tp_t, tp_i)
        for r in range(tp_i):
            plan = build_plan(cfg, RankLayout(world, tp=tp_t) if world != tp_t else train, tp_i, r, tables, layers,
                              lambda rank: 0, esz=4)
            dst = torch.zeros(plan.nbytes, dtype=torch.uint8)
            execute_plan_torch(plan, buffers, dst)
            w = weights_from_buffer(cfg, tp_i, r, plan, dst, torch.float32)
            for li in range(cfg.num_layers):
                p = f"decoder.layers.{li}."
                want_qkv = C.shard_qkv(merged[p + "self_attention.linear_qkv"], cfg.num_query_groups, tp_i, r)
                want_proj = C.shard_cols(merged[p + "self_attention.linear_proj"], tp_i, r)
                g, u = merged[p + "mlp.linear_fc1"].chunk(2, 0)
                want_fc1 = C.shard_fc1(g, u, tp_i, r)
                want_fc2 = C.shard_cols(merged[p + "mlp.linear_fc2"], tp_i, r)
                for got, want in ((w.layers[li].qkv_w, want_qkv), (w.layers[li].o_w, want_proj),
                                  (w.layers[li].gate_up_w, want_fc1), (w.layers[li].down_w, want_fc2)):
                    assert torch.allclose(got, want, atol=1e-6), (tp_i, r, li)


def test_plan_mixes_element_sizes_and_buffers():
    """A bf16 model whose routers stay fp32 in a flat buffer of their own: the plan addresses both buffers and
    sizes every tensor by its own element size."""
    from mindspeed_rl_b200.reshard.planner import ExpertPlacement

    cfg = _moe_cfg()
    full = GPTModel(cfg, seed=9).state_dict()
    e, ep_t = cfg.num_experts, 2
    train = RankLayout(2, ep=ep_t)
    layers = stage_layers(cfg.num_layers, 1)
    sources, table = {}, None
    for r in range(2):
        st = _expert_shard(full, cfg, ep_t, train.expert_coords(r)["ep"])
        main = {k: v.to(torch.bfloat16) for k, v in st.items() if not k.endswith("router.weight")}
        fp32 = {k: v for k, v in st.items() if k.endswith("router.weight")}
        slots, off, chunks = {}, 0, []
        for k, v in main.items():
            slots[k] = Slot(off, tuple(v.shape), 0)
            chunks.append(v.reshape(-1))
            off += v.numel()
        sources[(r, 0)] = torch.cat(chunks).contiguous().view(torch.uint8)
        off, chunks = 0, []
        for k, v in fp32.items():
            slots[k] = Slot(off, tuple(v.shape), 1, 4)
            chunks.append(v.reshape(-1))
            off += v.numel()
        sources[(r, 1)] = torch.cat(chunks).contiguous().view(torch.uint8)
        table = slots
    hosted = lambda layer: list(range(e))                      # every rollout rank hosts all experts
    src = lambda ep_index, stage: train.rank_of(dp=ep_index)
    for r in range(2):
        plan = build_plan(cfg, train, 1, r, [table], layers, lambda rank, buf=0: 0, esz=2,
                          experts=ExpertPlacement(e // ep_t, hosted, src))
        assert plan.desc_buf is not None and plan.esz_of
        dst = torch.zeros(plan.nbytes, dtype=torch.uint8)
        execute_plan_torch(plan, sources, dst)
        w = weights_from_buffer(cfg, 1, 0, plan, dst, torch.bfloat16,
                                moe_builder=lambda li, t: (t(f"decoder.layers.{li}.mlp.router.weight"),
                                                           t(f"decoder.layers.{li}.mlp.experts.weight1")))
        for li in range(cfg.num_layers):
            router, w1 = w.layers[li].moe
            assert router.dtype == torch.float32 and torch.equal(router, full[f"decoder.layers.{li}.mlp.router.weight"])
            assert w1.dtype == torch.bfloat16 and torch.equal(
                w1, full[f"decoder.layers.{li}.mlp.experts.weight1"].to(torch.bfloat16))


def test_plan_for_expert_recipe_layout_with_experts_spread_over_tp():
    """The 30B-A3B recipe's shape: train TP4 x EP2 with the experts spread over TP x EP (8 expert shards, expert
    TP 1), rollout TP1 x EP8: dense weights are gathered over TP, every rollout rank ends up with its block of
    experts, whichever training rank held them."""
    from mindspeed_rl_b200.reshard.planner import ExpertPlacement

    cfg = _moe_cfg()
    full = GPTModel(cfg, seed=9).state_dict()
    world, tp_t, ep_t, ep_i = 8, 4, 2, 8
    train = RankLayout(world, tp=tp_t, ep=ep_t, moe_tp_extend_ep=True)
    assert train.ep_total == 8 and train.expert_tp == 1
    layers = stage_layers(cfg.num_layers, 1)
    h, f, e = cfg.hidden_size, cfg.moe_ffn_hidden_size, cfg.num_experts
    buffers, tables = {}, [None]
    for r in range(world):
        c, ec = train.coords(r), train.expert_coords(r)
        st = _shard(_expert_shard(full, cfg, train.ep_total, ec["ep"]), cfg, tp_t, c["tp"])
        slots, flat = _flatten(_stage_state(st, layers[0], True, True))
        tables[0] = slots
        buffers[r] = flat.view(torch.uint8)
    infer = RankLayout(world, ep=ep_i)
    for r in range(world):
        ei = infer.expert_coords(r)["ep"]
        mine = train.expert_coords(r)
        per = e // ep_i

        def hosted(layer, ei=ei):
            return list(range(ei * per, (ei + 1) * per))

        def src_rank(ep_index, stage, mine=mine):
            stage_rank = mine["etp"] + train.expert_tp * (ep_index + train.ep_total * mine["edp"])
            return train.rank_of(tp=stage_rank % train.tp, cp=(stage_rank // train.tp) % train.cp,
                                 dp=stage_rank // (train.tp * train.cp), pp=stage)

        plan = build_plan(cfg, train, 1, r, tables, layers, lambda rank: 0, esz=4,
                          experts=ExpertPlacement(e // train.ep_total, hosted, src_rank))
        dst = torch.zeros(plan.nbytes, dtype=torch.uint8)
        execute_plan_torch(plan, buffers, dst)
        want = _shard(full, cfg, 1, 0)
        for name, (off, shape) in plan.tensors.items():
            if ".experts." in name:
                layer = int(name.split(".")[2])
                ids = hosted(layer)
                key = f"decoder.layers.{layer}.mlp.experts."
                ref = (full[key + "weight1"].view(h, e, 2 * f)[:, ids] if name.endswith("weight1")
                       else full[key + "weight2"].view(e, f, h)[ids]).reshape(shape)
            else:
                ref = want[name]
            got = dst[off:off + ref.numel() * 4].view(torch.float32).view(shape)
            assert torch.equal(got, ref), (r, name)



@pytest.mark.parametrize("tp_t,pp_t,tp_i,world", [(2, 2, 1, 4), (4, 1, 2, 4), (1, 2, 2, 4)])
def test_plan_for_latent_attention(tp_t, pp_t, tp_i, world):
    """Latent attention (DeepSeek-style): down-projections and their norms are replicated, up-projections are cut
    by heads, the output projection by columns; the rollout block built over the destination buffer computes
    the same q / k / v as a model that was sharded directly for the rollout layout."""
    from mindspeed_rl_b200.models.mla import MLASelfAttention
    cfg = _cfg(num_attention_heads=4, num_query_groups=4, kv_channels=None, add_qkv_bias=False,
               multi_latent_attention=True, q_lora_rank=24, kv_lora_rank=16, qk_head_dim=32, qk_pos_emb_head_dim=32,
               v_head_dim=64, max_position_embeddings=64)
    full = GPTModel(cfg, seed=3).state_dict()
    train = RankLayout(world, tp=tp_t, pp=pp_t)
    layers = stage_layers(cfg.num_layers, pp_t)
    buffers, tables = {}, [None] * pp_t
    for r in range(world):
        c = train.coords(r)
        st = _stage_state(_shard(full, cfg, tp_t, c["tp"]), layers[c["pp"]], c["pp"] == 0, c["pp"] == pp_t - 1)
        slots, flat = _flatten(st)
        tables[c["pp"]] = slots
        buffers[r] = flat.view(torch.uint8)
    x = torch.randn(5, cfg.hidden_size, generator=torch.Generator().manual_seed(0))
    pos = torch.arange(5)
    for r in range(world):
        plan = build_plan(cfg, train, tp_i, r, tables, layers, lambda rank: 0, esz=4)
        dst = torch.zeros(plan.nbytes, dtype=torch.uint8)
        execute_plan_torch(plan, buffers, dst)
        j = r % tp_i
        want = _shard(full, cfg, tp_i, j)
        assert set(plan.tensors) == set(want)
        for name, (off, shape) in plan.tensors.items():
            got = dst[off:off + want[name].numel() * 4].view(torch.float32).view(shape)
            assert torch.equal(got, want[name]), name
        w = weights_from_buffer(cfg, tp_i, j, plan, dst, torch.float32)
        assert w.layers[0].qkv_w is None and w.layers[0].mla is not None
        assert w.qkv_layout.num_heads == w.qkv_layout.num_kv_heads == 4 // tp_i and w.qkv_layout.head_dim == 64
        sa = "decoder.layers.1.self_attention."
        direct = MLASelfAttention.from_tensors(cfg, tp_i, {k[len(sa):]: v for k, v in want.items() if k.startswith(sa)})
        assert torch.equal(w.layers[1].mla.rollout_qkv(x, pos), direct.rollout_qkv(x, pos))
        assert torch.equal(w.layers[1].o_w, want[sa + "linear_proj.weight"])
        if tp_i == 1:                                     # and both equal the block of the unsharded model
            ref = GPTModel(cfg, seed=3).decoder.layers[1].self_attention
            assert torch.equal(w.layers[1].mla.rollout_qkv(x, pos), ref.rollout_qkv(x, pos))
