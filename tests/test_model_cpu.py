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


def test_lora_matches_merged_weights():
    """LoRA forward == forward with W + (alpha/r) B A; adapter gradients == chain rule through the
    merged-weight gradients; only adapters are trainable; adapters can be switched off."""
    from mindspeed_rl_b200.models import lora

    kw = dict(num_layers=2, hidden_size=32, ffn_hidden_size=64, num_attention_heads=4, num_query_groups=2,
              vocab_size=64, add_qkv_bias=True, params_dtype=torch.float32)
    targets = ("linear_qkv", "linear_proj", "linear_fc1", "linear_fc2")
    m = GPTModel(TransformerConfig(lora_r=4, lora_alpha=8, lora_target_modules=targets, **kw), device="cpu", seed=2)
    trainable = [n for n, p in m.named_parameters() if p.requires_grad]
    assert trainable and all(n.endswith(("lora_A", "lora_B")) for n in trainable)
    g = torch.Generator().manual_seed(7)
    for h in lora.holders(m):
        h.lora_B.data.normal_(0, 0.1, generator=g)
    plain = GPTModel(TransformerConfig(**kw), device="cpu", seed=2)
    sd = {k: v for k, v in m.state_dict().items() if "lora_" not in k}
    for name, h in [(n, mod) for n, mod in m.named_modules() if getattr(mod, "lora_A", None) is not None]:
        sd[name + ".weight"] = lora.merged_weight(h)
    plain.load_state_dict(sd)
    meta = PackedMeta.from_lengths([7, 12], "cpu")
    t = int(meta.cu_seqlens[-1])
    ids, labels, w = torch.randint(0, 64, (t,), generator=g), torch.randint(0, 64, (t,), generator=g), torch.randn(t, generator=g)
    lp, _ = m.forward_logprob(ids, labels, meta, 1.0, False)
    lp_ref, _ = plain.forward_logprob(ids, labels, meta, 1.0, False)
    assert torch.allclose(lp, lp_ref, atol=1e-5)
    (lp * w).sum().backward()
    (lp_ref * w).sum().backward()
    ref_mods = dict(plain.named_modules())
    for name, h in [(n, mod) for n, mod in m.named_modules() if getattr(mod, "lora_A", None) is not None]:
        dw = ref_mods[name].weight.grad
        s = h.lora_scale
        assert torch.allclose(h.lora_A.grad, s * h.lora_B.data.t() @ dw, atol=1e-5), name
        assert torch.allclose(h.lora_B.grad, s * dw @ h.lora_A.data.t(), atol=1e-5), name
        assert h.weight.grad is None
    with lora.adapter_disabled(m), torch.no_grad():
        off, _ = m.forward_logprob(ids, labels, meta, 1.0, False)
    base = GPTModel(TransformerConfig(**kw), device="cpu", seed=2)
    base.load_state_dict({k: v for k, v in m.state_dict().items() if "lora_" not in k})
    with torch.no_grad():
        want, _ = base.forward_logprob(ids, labels, meta, 1.0, False)
    assert torch.allclose(off, want, atol=1e-6) and not torch.allclose(off, lp.detach(), atol=1e-4)


def test_swap_attention_gives_identical_gradients():
    """Activation offload between forward and backward changes nothing numerically; with block
    recompute it only touches the layers that keep their intermediates."""
    from mindspeed_rl_b200.models import activation_swap
    from mindspeed_rl_b200.models.gpt import GPTModel, PackedMeta
    from mindspeed_rl_b200.models.transformer_config import TransformerConfig
    kw = dict(num_layers=3, hidden_size=64, ffn_hidden_size=128, num_attention_heads=4, num_query_groups=2,
              vocab_size=96, params_dtype=torch.float32, max_position_embeddings=128,
              recompute_granularity="full", recompute_method="block", recompute_num_layers=1)
    lens = [40, 23]
    meta = PackedMeta.from_lengths(lens, "cpu")
    t = sum(lens)
    ids, labels = torch.randint(0, 96, (t,)), torch.randint(0, 96, (t,))
    grads = []
    for swap in (False, True):
        m = GPTModel(TransformerConfig(swap_attention=swap, **kw), device="cpu", seed=4)
        sw = activation_swap.swapper_for("cpu")
        sw.min_bytes, sw.bytes_out, sw.bytes_in = 1024, 0, 0
        lp, _ = m.forward_logprob(ids, labels, meta)
        lp.sum().backward()
        grads.append({n: p.grad.clone() for n, p in m.named_parameters()})
        if swap:
            assert sw.bytes_out > 0 and sw.bytes_in == sw.bytes_out and sw.last is None
        else:
            assert sw.bytes_out == 0
    for n in grads[0]:
        assert torch.equal(grads[0][n], grads[1][n]), n
    # restricted to some parts of a layer: fewer bytes leave, gradients unchanged; unknown names are refused
    full_bytes = sw.bytes_out
    m = GPTModel(TransformerConfig(swap_attention=True, swap_modules=("self_attention",), **kw), device="cpu", seed=4)
    sw.bytes_out = sw.bytes_in = 0
    lp, _ = m.forward_logprob(ids, labels, meta)
    lp.sum().backward()
    assert 0 < sw.bytes_out < full_bytes and sw.bytes_in == sw.bytes_out
    for n, p_ in m.named_parameters():
        assert torch.equal(grads[0][n], p_.grad), n
    import pytest
    with pytest.raises(ValueError):
        activation_swap.keys_of(("attention_core",))
