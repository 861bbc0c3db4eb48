"""MoE layer (hand-written expert backward + autograd router) against a dense autograd oracle,
MoE rollout equivalence, and checkpoint / HF-converter round trips."""
import os
import tempfile
from types import SimpleNamespace

import torch

from mindspeed_rl_b200.checkpoint import convert as C
from mindspeed_rl_b200.checkpoint.mcore import load_checkpoint, save_checkpoint
from mindspeed_rl_b200.models.gpt import GPTModel, PackedMeta
from mindspeed_rl_b200.models.moe import route
from mindspeed_rl_b200.models.transformer_config import TransformerConfig
from mindspeed_rl_b200.optim.distributed_optimizer import DistributedOptimizer, OptimizerParamScheduler
from mindspeed_rl_b200.parallel.ddp import DistributedDataParallel
from mindspeed_rl_b200.reshard.alias import alias_rollout_weights
from mindspeed_rl_b200.rollout.engine import LLMEngine
from mindspeed_rl_b200.rollout.scheduler import SamplingParams


def moe_cfg(**kw):
    base = dict(num_layers=2, hidden_size=32, ffn_hidden_size=64, num_attention_heads=4, num_query_groups=2,
                vocab_size=96, params_dtype=torch.float32, max_position_embeddings=128, num_experts=8,
                moe_router_topk=2, moe_ffn_hidden_size=16, norm_topk_prob=True, moe_aux_loss_coeff=0.01,
                recompute_granularity="full")
    base.update(kw)
    return TransformerConfig(**base)


def test_moe_layer_gradients_match_autograd():
    torch.manual_seed(0)
    cfg = moe_cfg()
    m = GPTModel(cfg, device="cpu")
    lens = [7, 5]
    meta = PackedMeta.from_lengths(lens, "cpu")
    t = sum(lens)
    ids, labels = torch.randint(0, 96, (t,)), torch.randint(0, 96, (t,))
    logp, _ = m.forward_logprob(ids, labels, meta)
    w = torch.randn(t)
    (logp * w).sum().backward()
    got = {n: p.grad.clone() for n, p in m.named_parameters()}

    # oracle: same math with plain autograd
    sd = {n: p.detach().clone().requires_grad_(True) for n, p in m.named_parameters()}
    hd, nh, nkv, rep = cfg.head_dim, 4, 2, 2
    rms = lambda x, g: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.norm_epsilon) * g
    pos = meta.positions.long()
    inv = 1.0 / (cfg.rotary_base ** (torch.arange(0, hd // 2).double() * 2 / hd))
    ang = (pos.double()[:, None] * inv[None]).float()
    cos, sin = ang.cos()[:, None], ang.sin()[:, None]
    rope = lambda x: torch.cat([x[..., :hd // 2] * cos - x[..., hd // 2:] * sin,
                                x[..., hd // 2:] * cos + x[..., :hd // 2] * sin], -1)
    h = sd["embedding.word_embeddings.weight"][ids]
    aux_total = 0
    for i in range(2):
        p = f"decoder.layers.{i}."
        x = rms(h, sd[p + "input_layernorm.weight"])
        qkv = x @ sd[p + "self_attention.linear_qkv.weight"].t()
        g = qkv.view(t, nkv, rep + 2, hd)
        q, k, v = rope(g[:, :, :rep].reshape(t, nh, hd)), rope(g[:, :, rep]), g[:, :, rep + 1]
        outs, cu = [], meta.cu_seqlens.tolist()
        for b in range(len(lens)):
            s, e = cu[b], cu[b + 1]
            o = torch.nn.functional.scaled_dot_product_attention(
                q[s:e].transpose(0, 1), k[s:e].transpose(0, 1).repeat_interleave(rep, 0),
                v[s:e].transpose(0, 1).repeat_interleave(rep, 0), is_causal=True)
            outs.append(o.transpose(0, 1).reshape(e - s, nh * hd))
        h = h + torch.cat(outs) @ sd[p + "self_attention.linear_proj.weight"].t()
        x = rms(h, sd[p + "pre_mlp_layernorm.weight"])
        logits = x.float() @ sd[p + "mlp.router.weight"].t()
        top_p, top_i, scores = route(logits, cfg)
        f = torch.zeros(8).scatter_add_(0, top_i.reshape(-1), torch.ones(top_i.numel())) / (t * 2)
        aux_total = aux_total + 0.01 * 8 * (f * scores.mean(0)).sum()
        w1 = sd[p + "mlp.experts.weight1"].view(32, 8, 32)
        w2 = sd[p + "mlp.experts.weight2"].view(8, 16, 32)
        out = torch.zeros_like(x)
        for tok in range(t):
            for j in range(2):
                e_ = int(top_i[tok, j])
                gu = x[tok] @ w1[:, e_]
                out[tok] = out[tok] + top_p[tok, j] * ((torch.nn.functional.silu(gu[:16]) * gu[16:]) @ w2[e_])
        h = h + out
    x = rms(h, sd["decoder.final_layernorm.weight"])
    ls = torch.log_softmax(x @ sd["output_layer.weight"].t(), -1)
    ((ls.gather(-1, labels[:, None])[:, 0] * w).sum() + aux_total).backward()
    for n in got:
        ref = sd[n].grad
        err = (got[n] - ref).abs().max() / (ref.abs().max() + 1e-9)
        assert err < 2e-4, (n, float(err))


def test_moe_rollout_matches_training_forward():
    torch.manual_seed(1)
    cfg = moe_cfg()
    m = GPTModel(cfg, device="cpu")
    for p in m.parameters():
        p.data.mul_(4.0)
    eng = LLMEngine(cfg, "cpu", max_num_seqs=4, max_num_batched_tokens=64, max_model_len=32, block_size=4)
    eng.runner.bind_weights(alias_rollout_weights(m))
    eng.init_cache(32)
    prompt = [3, 9, 27, 81, 5]
    out = eng.generate([prompt], SamplingParams(n=1, temperature=0.0, max_tokens=5))[0].outputs[0].token_ids
    ids = list(prompt)
    for _ in range(5):
        with torch.no_grad():
            lg = m.forward_logits(torch.tensor(ids), PackedMeta.from_lengths([len(ids)], "cpu"))
        ids.append(int(lg[-1].argmax()))
    assert out == ids[len(prompt):]


def test_mcore_checkpoint_round_trip():
    torch.manual_seed(2)
    cfg = TransformerConfig(num_layers=2, hidden_size=32, ffn_hidden_size=64, num_attention_heads=4,
                            num_query_groups=2, vocab_size=64, add_qkv_bias=True, params_dtype=torch.float32)
    m = DistributedDataParallel(GPTModel(cfg, device="cpu"))
    opt = DistributedOptimizer(m.buffers, lr=1e-3)
    sch = OptimizerParamScheduler(opt, 1e-3)
    for b in m.buffers:
        b.grad_data.normal_()
    opt.step()
    sch.step(5)
    with tempfile.TemporaryDirectory() as d:
        mc = SimpleNamespace(dict=lambda: {"hidden_size": 32}, finetune=False, no_load_optim=False, no_load_rng=False)
        rank_dir = save_checkpoint(d, 7, m.module, opt, sch, config=mc, consumed_train_samples=56)
        assert os.path.isfile(os.path.join(d, "latest_checkpointed_iteration.txt"))
        assert rank_dir.endswith(os.path.join("iter_0000007", "mp_rank_00"))
        m2 = DistributedDataParallel(GPTModel(cfg, device="cpu", seed=99))
        opt2 = DistributedOptimizer(m2.buffers, lr=1e-3)
        sch2 = OptimizerParamScheduler(opt2, 1e-3)
        it, consumed = load_checkpoint(d, m2.module, opt2, sch2, config=mc)
        assert (it, consumed) == (7, 56)
        for (n, a), (_, b) in zip(m.module.state_dict().items(), m2.module.state_dict().items()):
            assert torch.equal(a, b), n
        assert torch.equal(opt.state[0]["exp_avg"], opt2.state[0]["exp_avg"]) and opt2.step_count == 1
        assert sch2.num_steps == sch.num_steps


def test_hf_mcore_conversion_round_trip_with_tp_pp():
    torch.manual_seed(3)
    ns = SimpleNamespace(num_layers=4, hidden_size=32, num_attention_heads=4, num_query_groups=2, kv_channels=8,
                         num_experts=None, untie_embeddings_and_output_weights=True, moe_ffn_hidden_size=None)
    hf = {"model.embed_tokens.weight": torch.randn(64, 32), "model.norm.weight": torch.randn(32),
          "lm_head.weight": torch.randn(64, 32)}
    for i in range(4):
        p = f"model.layers.{i}."
        hf.update({p + "input_layernorm.weight": torch.randn(32), p + "post_attention_layernorm.weight": torch.randn(32),
                   p + "self_attn.q_proj.weight": torch.randn(32, 32), p + "self_attn.k_proj.weight": torch.randn(16, 32),
                   p + "self_attn.v_proj.weight": torch.randn(16, 32), p + "self_attn.o_proj.weight": torch.randn(32, 32),
                   p + "self_attn.q_proj.bias": torch.randn(32), p + "self_attn.k_proj.bias": torch.randn(16),
                   p + "self_attn.v_proj.bias": torch.randn(16), p + "mlp.gate_proj.weight": torch.randn(48, 32),
                   p + "mlp.up_proj.weight": torch.randn(48, 32), p + "mlp.down_proj.weight": torch.randn(32, 48)})
    with tempfile.TemporaryDirectory() as d:
        shards = C.hf_to_mcore(hf, ns, tp=2, pp=2)
        C.write_mcore(shards, d, 2, 2, 1)
        back = C.mcore_to_hf(C.read_mcore(d, 2, 2), ns, tp=2, pp=2)
        assert set(back) == set(hf)
        for k in hf:
            assert torch.equal(back[k], hf[k]), k
        C.save_hf_state(back, os.path.join(d, "hf"))
        again = C.load_hf_state(os.path.join(d, "hf"))
        assert all(torch.equal(again[k], hf[k]) for k in hf)
    # a TP-1 conversion loads into the model and reproduces HF-style attention layout
    cfg = TransformerConfig(num_layers=4, hidden_size=32, ffn_hidden_size=48, num_attention_heads=4,
                            num_query_groups=2, vocab_size=64, add_qkv_bias=True, params_dtype=torch.float32)
    model = GPTModel(cfg, device="cpu")
    missing, unexpected = model.load_state_dict(C.hf_to_mcore(hf, ns)[(0, 0, 0)], strict=False)
    assert not missing and not unexpected
