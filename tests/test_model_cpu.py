"""Model-level invariants on CPU: recompute modes give identical gradients."""
import torch

from mindspeed_rl_b200.models.gpt import GPTModel, PackedMeta
from mindspeed_rl_b200.models.transformer_config import TransformerConfig


def _grads(**kw):
    cfg = TransformerConfig(num_layers=3, hidden_size=32, ffn_hidden_size=64, num_attention_heads=4,
                            num_query_groups=2, vocab_size=64, add_qkv_bias=True, params_dtype=torch.float32, **kw)
    model = GPTModel(cfg, device="cpu", seed=2)
    meta = PackedMeta.from_lengths([7, 12], "cpu")
    t = int(meta.cu_seqlens[-1])
    g = torch.Generator().manual_seed(0)
    ids, labels, w = torch.randint(0, 64, (t,), generator=g), torch.randint(0, 64, (t,), generator=g), torch.randn(t, generator=g)
    lp, _ = model.forward_logprob(ids, labels, meta, 1.0, False)
    (lp * w).sum().backward()
    return lp.detach(), {n: p.grad.clone() for n, p in model.named_parameters()}, model


def test_recompute_modes_agree():
    lp0, g0, m0 = _grads(recompute_granularity=None)
    lp1, g1, m1 = _grads(recompute_granularity="full")
    lp2, g2, m2 = _grads(recompute_granularity="full", recompute_method="block", recompute_num_layers=1,
                         recompute_activation_function=True)
    assert [l.recompute_full for l in m2.decoder.layers] == [True, False, False]
    assert all(l.recompute_full for l in m1.decoder.layers)
    for lp, g in ((lp1, g1), (lp2, g2)):
        assert torch.allclose(lp, lp0, atol=1e-6)
        for n in g0:
            assert torch.allclose(g[n], g0[n], atol=1e-6), n
