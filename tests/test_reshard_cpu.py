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
    cfg = _cfg()
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
        assert w.layers[0].qkv_w.shape[0] == (cfg.num_attention_heads + 2 * cfg.num_query_groups) // tp_i * 16
        assert w.vocab_start == j * cfg.vocab_size // tp_i
