"""Multi-head latent attention: the block against an explicit per-sequence formulation, gradients of
the hand-written layer path against plain autograd, and a whole GRPO run of a shrunk DeepSeek-style
model (latent attention + routed / shared experts) including its rollout."""
import math

import torch

from mindspeed_rl_b200.models.gpt import GPTModel, PackedMeta
from mindspeed_rl_b200.models.transformer_config import TransformerConfig

KW = dict(num_layers=2, hidden_size=64, ffn_hidden_size=96, num_attention_heads=4, num_query_groups=4,
          vocab_size=96, params_dtype=torch.float32, max_position_embeddings=128, multi_latent_attention=True,
          q_lora_rank=24, kv_lora_rank=16, qk_head_dim=16, qk_pos_emb_head_dim=8, v_head_dim=16,
          recompute_granularity=None)


def test_mla_block_matches_explicit_attention():
    torch.manual_seed(0)
    m = GPTModel(TransformerConfig(**KW), device="cpu", seed=1)
    sa = m.decoder.layers[0].self_attention
    meta = PackedMeta.from_lengths([5, 9, 2], "cpu")
    t = int(meta.cu_seqlens[-1])
    x = torch.randn(t, 64)
    out = sa(x, meta)
    q, k, v = sa.qkv(x, meta.positions)
    want = torch.zeros(t, 4 * 16)
    cu = meta.cu_seqlens.tolist()
    for s, e in zip(cu[:-1], cu[1:]):
        for h in range(4):
            sc = (q[s:e, h].double() @ k[s:e, h].double().t()) * sa.softmax_scale
            sc = sc.masked_fill(torch.triu(torch.ones(e - s, e - s, dtype=torch.bool), 1), float("-inf"))
            want[s:e, h * 16:(h + 1) * 16] = (torch.softmax(sc, -1) @ v[s:e, h].double()).float()
    want = want @ sa.linear_proj.weight.t()
    assert torch.allclose(out, want, atol=1e-4), (out - want).abs().max()
    assert abs(sa.softmax_scale - 1 / math.sqrt(24)) < 1e-9
    # rotary part: the key's rotary slice is shared by all heads and position dependent
    assert torch.equal(k[:, 0, 16:], k[:, 3, 16:]) and not torch.allclose(k[0, 0, 16:], k[1, 0, 16:])


def test_mla_layer_gradients_match_autograd():
    """The layer keeps only the block's input and re-runs the block in its hand-written backward; the
    result must equal differentiating the same forward with autograd end to end."""
    torch.manual_seed(1)
    a = GPTModel(TransformerConfig(**KW), device="cpu", seed=2)
    meta = PackedMeta.from_lengths([7, 4], "cpu")
    t = int(meta.cu_seqlens[-1])
    ids, labels, w = torch.randint(0, 96, (t,)), torch.randint(0, 96, (t,)), torch.randn(t)
    (a.forward_logprob(ids, labels, meta, 1.0, False)[0] * w).sum().backward()
    got = {n: (p.grad if p.grad is not None else p.main_grad).clone() for n, p in a.named_parameters()}

    # the same computation written with plain differentiable operations
    b = GPTModel(TransformerConfig(**KW), device="cpu", seed=2)
    h = b.embedding.word_embeddings.weight[ids]
    rms = lambda x, wt: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * wt
    for layer in b.decoder.layers:
        h = h + layer.self_attention(rms(h, layer.input_layernorm.weight), meta)
        gu = rms(h, layer.pre_mlp_layernorm.weight) @ layer.mlp.linear_fc1.weight.t()
        g, u = gu.chunk(2, dim=-1)
        h = h + (torch.nn.functional.silu(g) * u) @ layer.mlp.linear_fc2.weight.t()
    z = rms(h, b.decoder.final_layernorm.weight) @ b.output_weight().t()
    lp = torch.log_softmax(z, -1).gather(-1, labels[:, None])[:, 0]
    (lp * w).sum().backward()
    for n, p in b.named_parameters():
        assert torch.allclose(got[n], p.grad, atol=2e-4, rtol=1e-3), (n, (got[n] - p.grad).abs().max())


def test_grpo_run_with_latent_attention_and_experts():
    from mindspeed_rl_b200.config import compose
    from mindspeed_rl_b200.runtime.launch import run_rl
    cfg = compose("grpo_tiny_cpu", None, [
        "+model.tiny_qwen2.multi_latent_attention=true", "+model.tiny_qwen2.q_lora_rank=48",
        "+model.tiny_qwen2.kv_lora_rank=32", "+model.tiny_qwen2.qk_head_dim=32",
        "+model.tiny_qwen2.qk_pos_emb_head_dim=32", "+model.tiny_qwen2.v_head_dim=64",
        "+model.tiny_qwen2.group_query_attention=false", "+model.tiny_qwen2.add_qkv_bias=false",
        "+model.tiny_qwen2.num_experts=4", "+model.tiny_qwen2.moe_router_topk=2",
        "+model.tiny_qwen2.moe_ffn_hidden_size=32", "+model.tiny_qwen2.n_shared_experts=1",
        "+model.tiny_qwen2.first_k_dense_replace=1", "+model.tiny_qwen2.moe_router_score_function=sigmoid",
        "+model.tiny_qwen2.norm_topk_prob=true"])
    hist = run_rl(cfg, "grpo")
    assert len(hist) == 2 and all("actor/pg_loss" in m and m["timing/rollout"] > 0 for m in hist)
    assert abs(hist[0]["actor/kl_loss"]) < 1e-4        # reference copy == actor before the first update


def test_latent_attention_checkpoint_round_trip_through_hf_names():
    """mcore (TP 2) -> Hugging Face names -> mcore: every tensor comes back bit-identical, the rotary
    rows are interleaved on the Hugging Face side, and a model loaded from the converted shards gives
    the single-rank model's outputs."""
    from mindspeed_rl_b200.checkpoint import convert as C
    cfg = TransformerConfig(**KW)
    full = GPTModel(cfg, device="cpu", seed=3)
    sd = {k: v.detach() for k, v in full.state_dict().items()}
    hf = C.mcore_to_hf({(0, 0, 0): sd}, cfg)
    assert "model.layers.0.self_attn.kv_a_proj_with_mqa.weight" in hf and "model.layers.1.self_attn.q_b_proj.weight" in hf
    a = hf["model.layers.0.self_attn.kv_a_proj_with_mqa.weight"][cfg.kv_lora_rank:]
    b = sd["decoder.layers.0.self_attention.linear_kv_down_proj.weight"][cfg.kv_lora_rank:]
    assert torch.equal(a[0::2], b[:4]) and torch.equal(a[1::2], b[4:])          # (even, odd) pairs <- halves
    shards = C.hf_to_mcore(hf, cfg, tp=2)
    back = C.mcore_to_hf(shards, cfg, tp=2)
    assert set(back) == set(hf) and all(torch.equal(back[k], hf[k]) for k in hf)
    one = C.hf_to_mcore(hf, cfg, tp=1)[(0, 0, 0)]
    assert set(one) == set(sd) and all(torch.equal(one[k], sd[k]) for k in sd)
