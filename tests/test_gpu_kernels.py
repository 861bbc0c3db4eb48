"""Numerics of every CUDA kernel against the plain PyTorch fp32 formulation of the same op.

Each test runs the op on CUDA tensors (kernel path) and on CPU copies (reference path inside the
same front-end) and compares within bf16 tolerances."""
import math

import pytest
import torch

from mindspeed_rl_b200 import ops
from mindspeed_rl_b200.ops import QKVLayout

pytestmark = pytest.mark.gpu
DEV = "cuda"


def close(a, b, atol, rtol, what=""):
    a, b = a.detach().float().cpu(), b.detach().float().cpu()
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    assert bool((err <= tol).all()), f"{what}: max err {err.max().item():.4g} (ref max {b.abs().max().item():.4g})"


@pytest.mark.parametrize("rows,h", [(2000, 3584), (1501, 4096), (900, 1024), (777, 2048)])
def test_rmsnorm_fwd_many_rows_warp_per_row(rows, h):
    """Enough rows for the warp-per-row forward (three row widths of its template, with and without the
    fused residual add) against the fp32 formulation."""
    torch.manual_seed(1)
    x = torch.randn(rows, h, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(rows, h, device=DEV, dtype=torch.bfloat16)
    w = (1 + 0.1 * torch.randn(h, device=DEV)).bfloat16()
    for r in (None, res):
        y, rstd, s = ops.rmsnorm_fwd(x, w, 1e-6, residual=r)
        xs = x.float() if r is None else (x.float() + r.float()).bfloat16().float()
        want_rstd = torch.rsqrt(xs.pow(2).mean(-1) + 1e-6)
        close(rstd, want_rstd, 1e-3, 1e-2, "rstd")
        close(y, (xs * want_rstd[:, None] * w.float()).bfloat16(), 2e-2, 2e-2, "y")
        if r is not None:
            assert torch.equal(s, xs.bfloat16())


@pytest.mark.parametrize("rows,h", [(37, 3584), (5, 4096), (300, 256), (9, 5120)])
def test_rmsnorm_fwd_bwd(rows, h):
    torch.manual_seed(0)
    x = torch.randn(rows, h, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(rows, h, device=DEV, dtype=torch.bfloat16)
    w = (1 + 0.1 * torch.randn(h, device=DEV)).bfloat16()
    y, rstd, s = ops.rmsnorm_fwd(x, w, 1e-6, residual=res)
    yr, rstdr, sr = ops.rmsnorm_fwd(x.cpu(), w.cpu(), 1e-6, residual=res.cpu())
    close(s, sr, 1e-2, 1e-2, "sum")
    close(y, yr, 2e-2, 2e-2, "y")
    close(rstd, rstdr, 1e-3, 1e-2, "rstd")
    dy = torch.randn(rows, h, device=DEV, dtype=torch.bfloat16)
    dres = torch.randn(rows, h, device=DEV, dtype=torch.bfloat16)
    dw = torch.zeros(h, device=DEV, dtype=torch.float32)
    dx = ops.rmsnorm_bwd(dy, s, w, rstd, dw, dres=dres)
    dwr = torch.zeros(h, dtype=torch.float32)
    dxr = ops.rmsnorm_bwd(dy.cpu(), s.cpu(), w.cpu(), rstd.cpu(), dwr, dres=dres.cpu())
    close(dx, dxr, 3e-2, 3e-2, "dx")
    close(dw, dwr, 5e-2 * math.sqrt(rows), 2e-2, "dw")


@pytest.mark.parametrize("interleaved", [True, False])
def test_headnorm_and_rope(interleaved):
    torch.manual_seed(1)
    lay = QKVLayout(8, 2, 128, interleaved)
    t = 53
    qkv = torch.randn(t, lay.width, device=DEV, dtype=torch.bfloat16)
    w = (1 + 0.1 * torch.randn(128, device=DEV)).bfloat16()
    pos = torch.randint(0, 4000, (t,), device=DEV, dtype=torch.int32)
    tab = ops.rope_table(4096, 128, 1e6, DEV)
    a, b = qkv.clone(), qkv.cpu().clone()
    for which in ("q", "k"):
        r1 = ops.headnorm_fwd_(a, lay, which, w, 1e-6)
        r2 = ops.headnorm_fwd_(b, lay, which, w.cpu(), 1e-6)
        close(r1, r2, 1e-3, 1e-2, "rstd " + which)
    close(a, b, 3e-2, 2e-2, "headnorm")
    ops.rope_(a, lay, pos, tab)
    ops.rope_(b, lay, pos.cpu(), tab.cpu())
    close(a, b, 4e-2, 2e-2, "rope")
    # inverse rotation restores the input up to bf16 rounding
    c = a.clone()
    ops.rope_(c, lay, pos, tab, inverse=True)
    ref = qkv.clone()
    for which in ("q", "k"):
        ops.headnorm_fwd_(ref, lay, which, w, 1e-6)
    close(c, ref, 6e-2, 3e-2, "rope inverse")
    # head-norm backward
    dq = torch.randn(t, lay.width, device=DEV, dtype=torch.bfloat16)
    dqc = dq.cpu().clone()
    rs = ops.headnorm_fwd_(qkv.clone(), lay, "q", w, 1e-6)
    dw = torch.zeros(128, device=DEV)
    dwr = torch.zeros(128)
    ops.headnorm_bwd_(dq, qkv, lay, "q", w, rs, dw)
    ops.headnorm_bwd_(dqc, qkv.cpu(), lay, "q", w.cpu(), rs.cpu(), dwr)
    close(dq, dqc, 3e-2, 3e-2, "headnorm dx")
    close(dw, dwr, 0.3, 3e-2, "headnorm dw")


def test_swiglu_and_colsum():
    torch.manual_seed(2)
    x = torch.randn(77, 2 * 1536, device=DEV, dtype=torch.bfloat16)
    y = ops.swiglu_fwd(x)
    close(y, ops.swiglu_fwd(x.cpu()), 2e-2, 2e-2, "swiglu")
    dy = torch.randn(77, 1536, device=DEV, dtype=torch.bfloat16)
    close(ops.swiglu_bwd(x, dy), ops.swiglu_bwd(x.cpu(), dy.cpu()), 3e-2, 2e-2, "swiglu bwd")
    out = torch.zeros(3072, device=DEV)
    ops.colsum_accumulate(x, out)
    close(out, x.float().sum(0), 1e-2, 1e-3, "colsum")
    a, b = torch.randn(4096, device=DEV).bfloat16(), torch.randn(4096, device=DEV).bfloat16()
    close(ops.add(a, b), a.float() + b.float(), 2e-2, 1e-2, "add")


@pytest.mark.parametrize("hd,nh,nkv,interleaved", [(128, 4, 2, True), (64, 4, 4, False), (128, 7, 1, True)])
def test_flash_attention_varlen(hd, nh, nkv, interleaved):
    torch.manual_seed(3)
    lay = QKVLayout(nh, nkv, hd, interleaved)
    lens = [1, 70, 130, 64, 257]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    t = int(cu[-1])
    qkv = (0.5 * torch.randn(t, lay.width, device=DEV)).bfloat16()
    out, lse = ops.attn_varlen_fwd(qkv, lay, cu.to(DEV), max(lens))
    outr, lser = ops.attn_varlen_fwd(qkv.cpu(), lay, cu, max(lens))
    close(out, outr, 2e-2, 2e-2, "attn out")
    close(lse, lser, 2e-2, 1e-2, "lse")
    dout = (0.5 * torch.randn(t, nh * hd, device=DEV)).bfloat16()
    dqkv = ops.attn_varlen_bwd(dout, qkv, out, lse, lay, cu.to(DEV), max(lens))
    dqkvr = ops.attn_varlen_bwd(dout.cpu(), qkv.cpu(), outr, lser, lay, cu, max(lens))
    close(dqkv, dqkvr, 3e-2, 5e-2, "dqkv")


def test_flash_attention_prefix():
    torch.manual_seed(4)
    lay = QKVLayout(4, 2, 128, False)
    qlens, klens = [5, 64, 1], [40, 200, 65]
    cu_q = torch.tensor([0, 5, 69, 70], dtype=torch.int32)
    cu_k = torch.tensor([0, 40, 240, 305], dtype=torch.int32)
    qkv = (0.5 * torch.randn(70, lay.width, device=DEV)).bfloat16()
    k = (0.5 * torch.randn(305, 2, 128, device=DEV)).bfloat16()
    v = (0.5 * torch.randn(305, 2, 128, device=DEV)).bfloat16()
    out, _ = ops.attn_varlen_fwd(qkv, lay, cu_q.to(DEV), 64, kv=(k, v), cu_seqlens_k=cu_k.to(DEV))
    outr, _ = ops.attn_varlen_fwd(qkv.cpu(), lay, cu_q, 64, kv=(k.cpu(), v.cpu()), cu_seqlens_k=cu_k)
    close(out, outr, 2e-2, 2e-2, "prefix attention")


@pytest.mark.parametrize("nh,nkv,hd,bs", [(28, 4, 128, 16), (8, 8, 64, 8), (16, 1, 128, 16)])
def test_paged_decode_and_cache(nh, nkv, hd, bs):
    torch.manual_seed(5)
    lay = QKVLayout(nh, nkv, hd, True)
    lens = [1, 17, 300, 1025, 64]
    b = len(lens)
    nblocks = sum((n + bs - 1) // bs for n in lens) + 3
    kc = torch.zeros(nblocks, bs, nkv, hd, device=DEV, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    perm = torch.randperm(nblocks).tolist()
    maxb = max((n + bs - 1) // bs for n in lens)
    bt = torch.zeros(b, maxb, dtype=torch.int32)
    cur = 0
    for i, n in enumerate(lens):
        nb = (n + bs - 1) // bs
        bt[i, :nb] = torch.tensor(perm[cur:cur + nb], dtype=torch.int32)
        cur += nb
    # fill the cache through the write kernel, sequence by sequence
    for i, n in enumerate(lens):
        x = (0.5 * torch.randn(n, lay.width, device=DEV)).bfloat16()
        pos = torch.arange(n)
        slots = (bt[i, (pos // bs)].long() * bs + pos % bs).to(DEV)
        ops.kv_cache_write(x, lay, slots, kc, vc)
    kcr, vcr = kc.cpu(), vc.cpu()
    q = (0.5 * torch.randn(b, lay.width, device=DEV)).bfloat16()
    ctx = torch.tensor(lens, dtype=torch.int32)
    out = ops.paged_decode_attention(q, lay, kc, vc, bt.to(DEV), ctx.to(DEV), max(lens))
    outr = ops.paged_decode_attention(q.cpu(), lay, kcr, vcr, bt, ctx, max(lens))
    close(out, outr, 2e-2, 2e-2, "paged decode")
    # gather
    tok_seq = torch.tensor([2] * 300 + [4] * 64, dtype=torch.int32)
    tok_pos = torch.tensor(list(range(300)) + list(range(64)), dtype=torch.int32)
    kg, vg = ops.kv_cache_gather(kc, vc, bt.to(DEV), tok_seq.to(DEV), tok_pos.to(DEV))
    kgr, vgr = ops.kv_cache_gather(kcr, vcr, bt, tok_seq, tok_pos)
    assert torch.equal(kg.cpu(), kgr) and torch.equal(vg.cpu(), vgr)


@pytest.mark.parametrize("nh,nkv,hd,bs,n_samples,prompt", [(28, 4, 128, 16, 8, 200), (8, 2, 64, 16, 5, 70),
                                                           (16, 16, 128, 32, 8, 33), (28, 4, 128, 16, 8, 1100),
                                                           (8, 2, 64, 24, 5, 100)])
def test_paged_decode_shared_prefix(nh, nkv, hd, bs, n_samples, prompt):
    """Groups of samples share their prompt blocks; the grouped kernels (prefix read once per
    group + per-sample suffix + merge) must equal the plain per-sequence path."""
    torch.manual_seed(11)
    lay = QKVLayout(nh, nkv, hd, True)
    n_prompts = 3
    shared_blocks = prompt // bs                       # full prompt blocks are physically shared
    gen = [[1 + 37 * j + 11 * g for j in range(n_samples)] for g in range(n_prompts)]   # generated so far
    lens = [prompt + gen[g][j] for g in range(n_prompts) for j in range(n_samples)] + [90]   # + a singleton
    b = len(lens)
    maxb = max((n + bs - 1) // bs for n in lens)
    nblocks = b * maxb + 8
    kc = torch.zeros(nblocks, bs, nkv, hd, device=DEV, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    free = torch.randperm(nblocks).tolist()
    bt = torch.zeros(b, maxb, dtype=torch.int32)
    row = 0
    for g in range(n_prompts):
        prompt_kv = (0.5 * torch.randn(prompt, lay.width, device=DEV)).bfloat16()
        shared = [free.pop() for _ in range(shared_blocks)]
        for j in range(n_samples):
            n = lens[row]
            nb = (n + bs - 1) // bs
            blocks = shared + [free.pop() for _ in range(nb - shared_blocks)]
            bt[row, :nb] = torch.tensor(blocks, dtype=torch.int32)
            x = torch.cat([prompt_kv, (0.5 * torch.randn(n - prompt, lay.width, device=DEV)).bfloat16()])
            pos = torch.arange(n)
            ops.kv_cache_write(x, lay, (bt[row, pos // bs].long() * bs + pos % bs).to(DEV), kc, vc)
            row += 1
    n = lens[row]
    nb = (n + bs - 1) // bs
    bt[row, :nb] = torch.tensor([free.pop() for _ in range(nb)], dtype=torch.int32)
    pos = torch.arange(n)
    ops.kv_cache_write((0.5 * torch.randn(n, lay.width, device=DEV)).bfloat16(), lay,
                       (bt[row, pos // bs].long() * bs + pos % bs).to(DEV), kc, vc)
    q = (0.5 * torch.randn(b, lay.width, device=DEV)).bfloat16()
    ctx = torch.tensor(lens, dtype=torch.int32, device=DEV)
    btd = bt.to(DEV)
    plain = ops.paged_decode_attention(q, lay, kc, vc, btd, ctx, max(lens))
    ids = [g for g in range(n_prompts) for _ in range(n_samples)] + ["solo"]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    ref = ops.paged_decode_attention(q.cpu(), lay, kc.cpu(), vc.cpu(), bt, ctx.cpu(), max(lens))
    # the mma.sync shared pass (any prefix), then the tcgen05 one where it covers the shape (prefix rounded
    # down to its key tile, the rest read per sequence; group tables cut to the groups that have members)
    for tile in sorted({0, ops.decode_prefix_tile(nh, nkv, hd, bs)}):
        ks, rows, pre, shared_any = ops.build_decode_groups(ids, [prompt] * (b - 1) + [90],
                                                            ops.decode_group_max(nh, nkv, tile), multiple=max(1, tile))
        assert sorted(r for grp in rows for r in grp if r >= 0) == list(range(b))
        assert shared_any == (prompt >= max(1, tile)) and all(x % max(1, tile) == 0 for x in pre)
        real = sum(1 for grp in rows if grp[0] >= 0)
        grouped = ops.paged_decode_attention(q, lay, kc, vc, btd, ctx, max(lens),
                                             groups=(i32(ks), i32(rows[:real]), i32(pre[:real])), prefix_tile=tile)
        close(grouped, plain, 1e-2, 1e-2, f"shared-prefix decode (tile {tile})")
        close(grouped, ref, 2e-2, 2e-2, f"shared-prefix decode vs reference (tile {tile})")
        for splits in (1, 3):
            again = ops.paged_decode_attention(q, lay, kc, vc, btd, ctx, max(lens), prefix_splits=splits,
                                               groups=(i32(ks), i32(rows), i32(pre)), prefix_tile=tile)
            close(again, plain, 1e-2, 1e-2, f"shared-prefix decode (tile {tile}, {splits} splits)")
    from mindspeed_rl_b200.ops import gemm as G
    G.check_status(DEV, "shared-prefix decode")


def test_lmhead_logprob_fwd_bwd():
    torch.manual_seed(6)
    t, h, v = 300, 256, 5000
    x = (torch.randn(t, h, device=DEV)).bfloat16()
    w = (0.05 * torch.randn(v, h, device=DEV)).bfloat16()
    y = torch.randint(0, v, (t,), device=DEV)
    logp, ent, lse = ops.lmhead_logprob_fwd(x, w, y, 1 / 0.7, chunk=128)
    z = (x.float() @ w.float().t()) / 0.7
    ls = torch.log_softmax(z, -1)
    close(logp, ls.gather(-1, y[:, None])[:, 0], 3e-2, 1e-2, "logp")
    close(ent, -(ls.exp() * ls).sum(-1), 3e-2, 1e-2, "entropy")
    dlogp = torch.randn(t, device=DEV)
    dent = 0.1 * torch.randn(t, device=DEV)
    dw = torch.zeros_like(w)
    dx = ops.lmhead_logprob_bwd(x, w, y, lse, ent, dlogp, dent, dw, 1 / 0.7, chunk=128)
    xr = x.float().requires_grad_(True)
    wr = w.float().requires_grad_(True)
    zr = (xr @ wr.t()) / 0.7
    lsr = torch.log_softmax(zr, -1)
    ((lsr.gather(-1, y[:, None])[:, 0] * dlogp).sum() + (-(lsr.exp() * lsr).sum(-1) * dent).sum()).backward()
    close(dx, xr.grad, 2e-2, 5e-2, "dx")
    close(dw, wr.grad, 5e-2, 5e-2, "dw")


def test_policy_value_loss_gae():
    torch.manual_seed(7)
    b, l = 64, 200
    lp = -torch.rand(b, l, device=DEV) * 3
    old = lp + 0.3 * torch.randn(b, l, device=DEV)
    ref = lp + 0.3 * torch.randn(b, l, device=DEV)
    adv = torch.randn(b, l, device=DEV)
    mask = (torch.rand(b, l, device=DEV) > 0.3).float()
    for kl in ("low_var_kl", "kl", "abs", "mse"):
        for token_level in (True, False):
            d, st = ops.policy_loss_fwd_bwd(lp, old, ref, adv, mask, 0.2, 0.28, 0.01, kl, token_level, 0.5)
            dr, sr = ops.policy_loss_fwd_bwd(lp.cpu(), old.cpu(), ref.cpu(), adv.cpu(), mask.cpu(), 0.2, 0.28,
                                             0.01, kl, token_level, 0.5)
            close(d, dr, 1e-6, 1e-3, f"dlogp {kl}")
            for k in ("pg_loss", "pg_clipfrac", "ppo_kl", "kl_loss"):
                close(st[k], sr[k], 1e-4, 1e-3, f"{k} {kl} {token_level}")
    v, vo, ret = torch.randn(b, l, device=DEV), torch.randn(b, l, device=DEV), torch.randn(b, l, device=DEV)
    dv, st = ops.value_loss_fwd_bwd(v, vo, ret, mask, 0.5)
    dvr, sr = ops.value_loss_fwd_bwd(v.cpu(), vo.cpu(), ret.cpu(), mask.cpu(), 0.5)
    close(dv, dvr, 1e-6, 1e-3, "dv")
    close(st["vf_loss"], sr["vf_loss"], 1e-4, 1e-3, "vf_loss")
    r = torch.randn(b, l, device=DEV)
    a1, r1 = ops.gae(r, v, mask, 0.99, 0.95)
    a2, r2 = ops.gae(r.cpu(), v.cpu(), mask.cpu(), 0.99, 0.95)
    close(a1, a2, 1e-3, 1e-3, "gae adv")
    close(r1, r2, 1e-3, 1e-3, "gae ret")
    sc = torch.randint(0, 2, (b,), device=DEV).float()
    close(ops.group_norm_advantage(sc, mask, 8), ops.group_norm_advantage(sc.cpu(), mask.cpu(), 8),
          1e-4, 1e-4, "group norm")


def test_adam_and_norm():
    torch.manual_seed(8)
    n = 100_003
    p = torch.randn(n, device=DEV)
    g = (0.1 * torch.randn(n, device=DEV)).bfloat16()
    m, v = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    p16 = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    pc, mc, vc = p.cpu().clone(), m.cpu().clone(), v.cpu().clone()
    ss = torch.zeros(1, device=DEV)
    ops.sumsq_accumulate(g, ss)
    close(ss, g.float().pow(2).sum().reshape(1), 1e-2, 1e-3, "sumsq")
    coef, norm = torch.ones(1, device=DEV), torch.zeros(1, device=DEV)
    ops.clip_coefficient(ss, 1.0, 1.0, coef, norm)
    close(norm, ss.sqrt(), 1e-3, 1e-4, "norm")
    for step in (1, 2, 3):
        ops.adamw_step(p, m, v, g, p16, 1e-3, 0.9, 0.95, 1e-8, 0.01, step, coef)
        ops.adamw_step(pc, mc, vc, g.cpu(), None, 1e-3, 0.9, 0.95, 1e-8, 0.01, step, coef.cpu())
    close(p, pc, 1e-5, 1e-4, "adam p")
    close(p16, pc, 1e-2, 1e-2, "adam p16")


def test_sampler_distribution_and_greedy():
    torch.manual_seed(9)
    b, v = 64, 2000
    logits = 2 * torch.randn(b, v, device=DEV)
    keys = torch.arange(b, device=DEV, dtype=torch.int64)
    temp0 = torch.zeros(b, device=DEV)
    tok, lp = ops.sample(logits, temp0, None, None, None, keys, 0)
    assert torch.equal(tok, logits.argmax(-1))
    close(lp, torch.log_softmax(logits, -1).gather(-1, tok[:, None])[:, 0], 1e-3, 1e-3, "greedy logprob")
    # empirical distribution of one row under temperature 1
    row = torch.tensor([2.0, 1.0, 0.0, -1.0] + [-30.0] * (v - 4), device=DEV)
    n = 4000
    tok, _ = ops.sample(row.expand(n, v).contiguous(), torch.ones(n, device=DEV), None, None, None,
                        torch.arange(n, device=DEV, dtype=torch.int64), 123)
    freq = torch.bincount(tok, minlength=v)[:4].float() / n
    want = torch.softmax(row[:4], 0)
    assert (freq.cpu() - want.cpu()).abs().max() < 0.03, (freq, want)
    # top-k = 2 keeps only the two best tokens, top-p small keeps the best
    tok, _ = ops.sample(row.expand(n, v).contiguous(), torch.ones(n, device=DEV),
                        torch.full((n,), 2, device=DEV, dtype=torch.int32), None, None,
                        torch.arange(n, device=DEV, dtype=torch.int64), 5)
    assert int(tok.max()) <= 1
    tok, _ = ops.sample(row.expand(n, v).contiguous(), torch.ones(n, device=DEV), None,
                        torch.full((n,), 0.5, device=DEV), None,
                        torch.arange(n, device=DEV, dtype=torch.int64), 5)
    assert int(tok.max()) == 0
    # forced EOS probability
    tok, _ = ops.sample(row.expand(n, v).contiguous(), torch.ones(n, device=DEV), None, None, None,
                        torch.arange(n, device=DEV, dtype=torch.int64), 7,
                        eos_prob=torch.full((n,), 0.25, device=DEV), eos_id=1999)
    assert abs(float((tok == 1999).float().mean()) - 0.25) < 0.03


def test_swap_attention_and_reuse_fp32_param_on_gpu():
    """Activation offload through pinned memory and a side stream leaves the gradients unchanged;
    the residual-only optimizer follows the fp32-master one on the device kernels."""
    from mindspeed_rl_b200.models import activation_swap
    from mindspeed_rl_b200.models.gpt import GPTModel, PackedMeta
    from mindspeed_rl_b200.models.transformer_config import TransformerConfig
    from mindspeed_rl_b200.optim.distributed_optimizer import DistributedOptimizer
    from mindspeed_rl_b200.parallel.ddp import DistributedDataParallel
    kw = dict(num_layers=4, hidden_size=256, ffn_hidden_size=512, num_attention_heads=4, num_query_groups=2,
              vocab_size=512, kv_channels=64, max_position_embeddings=2048, recompute_granularity="full",
              recompute_method="block", recompute_num_layers=1)
    lens = [700, 523]
    meta = PackedMeta.from_lengths(lens, DEV)
    t = sum(lens)
    g = torch.Generator(device=DEV).manual_seed(2)
    ids = torch.randint(0, 512, (t,), device=DEV, generator=g)
    labels = torch.randint(0, 512, (t,), device=DEV, generator=g)
    grads = []
    for swap in (False, True):
        m = DistributedDataParallel(GPTModel(TransformerConfig(swap_attention=swap, **kw), device=DEV, seed=4))
        sw = activation_swap.swapper_for(DEV)
        sw.min_bytes, sw.bytes_out, sw.bytes_in = 64 << 10, 0, 0
        lp, _ = m.module.forward_logprob(ids, labels, meta)
        lp.sum().backward()
        torch.cuda.synchronize()
        grads.append([b.grad_data.float().clone() for b in m.buffers])
        assert (sw.bytes_out > 0) == swap and sw.bytes_in == sw.bytes_out
    for a, b in zip(*grads):
        # weight-gradient reductions use atomics, so two runs differ in the last bits; a lost or
        # early-reused activation would be off by far more
        assert (a - b).abs().max().item() <= 1e-2 * a.abs().max().item(), (a - b).abs().max().item()
    # optimizer: bf16 parameter + int16 residual against fp32 master weights
    outs = []
    for reuse in (False, True):
        m = DistributedDataParallel(GPTModel(TransformerConfig(**kw), device=DEV, seed=4))
        opt = DistributedOptimizer(m.buffers, lr=1e-3, weight_decay=0.1, clip_grad=1.0, reuse_fp32_param=reuse)
        for step in range(3):
            for b, gsrc in zip(m.buffers, grads[0]):
                b.grad_data.copy_(gsrc * (1 + step))
            opt.step()
        outs.append([b.param_data.float().clone() for b in m.buffers])
        full = opt.state_dict()["shards"][0]["master"]
        if reuse:
            torch.testing.assert_close(full, ref_master, rtol=1e-5, atol=1e-7)
        else:
            ref_master = full
    for a, b in zip(*outs):
        assert (a - b).abs().max() <= 2 ** -7 * a.abs().max()


def test_device_barrier_gives_up_when_a_peer_never_arrives():
    """The peer-memory barrier waits a bounded time for a flag; here nothing ever sets it (the
    "peer" is a second flag array in this GPU's own memory), so the kernel must come back with a
    status code and leave the context usable."""
    import ctypes
    import time

    from mindspeed_rl_b200.ops import _lib
    lib = _lib.load()
    flags = torch.zeros(2, 16, dtype=torch.int32, device=DEV)           # flag arrays of "rank 0" and "rank 1"
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ptrs = (ctypes.c_void_p * 2)(flags[0].data_ptr(), flags[1].data_ptr())
    epochs = (ctypes.c_uint * 2)(0, 1)
    t0 = time.time()
    rc = lib.msrl_symm_barrier(ptrs, ctypes.c_int(0), ctypes.c_int(2), epochs, ctypes.c_uint(0b10),
                               _lib.ptr(status), _lib.stream())
    assert rc == 0
    torch.cuda.synchronize()
    assert time.time() - t0 < 10.0
    assert int(status.item()) == 101                                    # gave up waiting for peer 1
    assert int(flags[1, 0].item()) == 1                                 # my arrival was published
    # the context still works, and a barrier whose flag is set passes at once
    flags[0, 1] = 2
    status.zero_()
    epochs = (ctypes.c_uint * 2)(0, 2)
    lib.msrl_symm_barrier(ptrs, ctypes.c_int(0), ctypes.c_int(2), epochs, ctypes.c_uint(0b10), _lib.ptr(status),
                          _lib.stream())
    torch.cuda.synchronize()
    assert int(status.item()) == 0


def test_attention_merge_kernel():
    """Folding a block result into the running (out, log-sum-exp) pair: kernel against the PyTorch
    formulation, whole-tensor and row-subset forms, including rows that saw no key on one side."""
    torch.manual_seed(8)
    t, nh, hd = 700, 6, 128
    for rows in (None, torch.randperm(t, device=DEV)[:333].sort().values):
        tb = t if rows is None else rows.numel()
        acc_o = torch.randn(t, nh, hd, device=DEV)
        acc_l = torch.randn(nh, t, device=DEV) * 3
        acc_l[0, :5] = float("-inf")
        acc_o[:5, 0] = 0
        o = torch.randn(tb, nh * hd, device=DEV).bfloat16()
        l = torch.randn(nh, tb, device=DEV) * 3
        ro, rl = acc_o.cpu().clone(), acc_l.cpu().clone()
        ops.attn_merge_(ro, rl, o.cpu(), l.cpu(), None if rows is None else rows.cpu())
        ops.attn_merge_(acc_o, acc_l, o, l, rows)
        close(acc_o, ro, 1e-4, 1e-4, "merged out")
        assert torch.equal(torch.isinf(acc_l).cpu(), torch.isinf(rl))      # rows no block touched keep -inf
        close(torch.nan_to_num(acc_l, neginf=0.0), torch.nan_to_num(rl, neginf=0.0), 1e-4, 1e-4, "merged lse")


def test_forward_backward_is_bit_reproducible():
    """Two runs of the same forward + backward give identical log-probs and identical gradient
    buffers: no result depends on the order in which atomics land (attention, norms with and without
    per-head norm, embedding gradient, LM head)."""
    from mindspeed_rl_b200.models.gpt import GPTModel, PackedMeta
    from mindspeed_rl_b200.models.transformer_config import TransformerConfig
    from mindspeed_rl_b200.optim.distributed_optimizer import DistributedOptimizer
    from mindspeed_rl_b200.parallel.ddp import DistributedDataParallel
    kw = dict(num_layers=2, hidden_size=512, ffn_hidden_size=1024, num_attention_heads=4, num_query_groups=2,
              vocab_size=2048, kv_channels=128, max_position_embeddings=4096, add_qkv_bias=True, qk_layernorm=True)
    lens = [700, 1523, 300]
    meta = PackedMeta.from_lengths(lens, DEV)
    t = sum(lens)
    g = torch.Generator(device=DEV).manual_seed(2)
    ids = torch.randint(0, 2048, (t,), device=DEV, generator=g)
    labels = torch.randint(0, 2048, (t,), device=DEV, generator=g)
    m = DistributedDataParallel(GPTModel(TransformerConfig(**kw), device=DEV, seed=4))
    opt = DistributedOptimizer(m.buffers, lr=1e-3, clip_grad=1.0)
    runs = []
    for _ in range(2):
        m.zero_grad_buffer()
        lp, _ = m.module.forward_logprob(ids, labels, meta)
        lp.sum().backward()
        norm = opt.compute_grad_norm().clone() if hasattr(opt, "compute_grad_norm") else None
        torch.cuda.synchronize()
        runs.append((lp.detach().clone(), [b.grad_data.clone() for b in m.buffers], opt._sumsq.clone()))
    assert torch.equal(runs[0][0], runs[1][0])
    for a, b in zip(runs[0][1], runs[1][1]):
        assert torch.equal(a, b)
    assert torch.equal(runs[0][2], runs[1][2])           # sum of squares of the gradients


def test_pack_tokens_and_unpack_response_kernels_match_reference():
    """K14: the device kernels against the PyTorch index arithmetic (exact equality), int32 and int64
    ids, ragged lengths, block padding, a stream padded at its end."""
    from mindspeed_rl_b200.ops.packing import pack_tokens, unpack_response
    torch.manual_seed(5)
    b, s = 37, 129
    p_len = torch.randint(1, 40, (b,), dtype=torch.int32)
    r_len = torch.randint(0, 89, (b,), dtype=torch.int32)
    ids2d = torch.randint(1, 150000, (b, s))
    lens = (p_len + r_len).long().clamp(max=s)
    padded = (lens + 7) // 8 * 8
    padded[-1] += 128
    cu = torch.zeros(b + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(padded, 0)
    total = int(cu[-1])
    want = pack_tokens(ids2d, p_len, r_len, cu, total)
    for dt in (torch.int64, torch.int32):
        got = pack_tokens(ids2d.to(dt).cuda(), p_len.cuda(), r_len.cuda(), cu.cuda(), total)
        for g, w in zip(got, want):
            assert torch.equal(g.cpu(), w)
    src = torch.randn(total)
    want_rows = unpack_response(src, cu, p_len, r_len, 96)
    got_rows = unpack_response(src.cuda(), cu.cuda(), p_len.cuda(), r_len.cuda(), 96)
    assert torch.equal(got_rows.cpu(), want_rows)
    got16 = unpack_response(src.bfloat16().cuda(), cu.cuda(), p_len.cuda(), r_len.cuda(), 96)
    assert torch.equal(got16.cpu(), unpack_response(src.bfloat16(), cu, p_len, r_len, 96))


def test_canary_pads_catch_a_write_past_the_output(monkeypatch):
    """Debug allocator: outputs carry pads of a known pattern; a write one element past the end is reported
    with the allocation site, an in-bounds write is not."""
    from mindspeed_rl_b200.ops import guard

    monkeypatch.setenv("MSRL_DEBUG_CANARY", "1")
    guard.check("before")
    x = torch.randn(37, 3584, device=DEV).bfloat16()
    w = torch.ones(3584, device=DEV).bfloat16()
    y, _, _ = ops.rmsnorm_fwd(x, w, 1e-6)                  # a real kernel writing a guarded output
    assert guard.check("rmsnorm") >= 1
    t = guard.empty(100, dtype=torch.float32, device=DEV)
    t.fill_(1.0)
    assert guard.check("inside") >= 1
    flat = torch.as_strided(t, (101,), (1,))               # one element past the end
    flat[100] = 7.0
    with pytest.raises(RuntimeError, match="after the tensor"):
        guard.check("past the end")
    del y, t, flat


@pytest.mark.parametrize("gdtype", [torch.bfloat16, torch.float32])
def test_embedding_grad_kernel_matches_fp32_sum(gdtype):
    """Rows of equal token ids are summed in fp32 in token order into the embedding gradient; run twice, the
    result is bit-identical."""
    from mindspeed_rl_b200.models.gpt import embedding_grad_accumulate

    torch.manual_seed(2)
    v, h, t = 500, 3584, 3000
    ids = torch.randint(0, 40, (t,), device=DEV)                 # many repeats per id
    ids[::7] = torch.randint(0, v, (len(ids[::7]),), device=DEV)
    d = torch.randn(t, h, device=DEV).bfloat16()
    g0 = torch.randn(v, h, device=DEV).to(gdtype)
    want = g0.float().clone()
    want.index_add_(0, ids, d.float())
    g1, g2 = g0.clone(), g0.clone()
    embedding_grad_accumulate(g1, ids, d)
    embedding_grad_accumulate(g2, ids, d)
    assert torch.equal(g1, g2)
    tol = 2e-2 if gdtype == torch.bfloat16 else 1e-3
    close(g1.float(), want, tol * want.abs().max().item(), tol, "embedding grad")
