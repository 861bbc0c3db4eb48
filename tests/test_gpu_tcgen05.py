"""tcgen05 / TMA GEMM and the fused LM-head statistics epilogue against PyTorch references."""
import pytest
import torch

from mindspeed_rl_b200.ops import gemm as G
from mindspeed_rl_b200.ops import _lib
from mindspeed_rl_b200.ops._lib import c_int, c_ll, ptr, stream

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (300, 520, 192), (1024, 3584, 3584), (77, 1000, 4096)])
def test_gemm_bf16_tn(m, n, k):
    torch.manual_seed(0)
    a = (torch.randn(m, k, device=DEV) * 0.5).bfloat16()
    b = (torch.randn(n, k, device=DEV) * 0.5).bfloat16()
    c = G.gemm_bf16_tn(a, b)
    G.check_status(DEV)
    _assert_close(c, a.float() @ b.float().t(), k)


def _assert_close(c, ref, k, scale=0.25):
    """bf16 output of an fp32-accumulated product of entries of magnitude ~``sqrt(scale)``: the result
    has standard deviation ``scale * sqrt(k)`` and carries one bf16 rounding (relative 2^-8), so the
    band is 1 % relative plus 1 % of that standard deviation."""
    err = (c.float() - ref).abs()
    tol = 1e-2 * ref.abs() + 1e-2 * scale * (k ** 0.5)
    assert bool((err <= tol).all()), f"max err {err.max().item()} ref max {ref.abs().max().item()}"


PAIR_SHAPES = [(256, 256, 64), (128, 256, 128), (300, 520, 192), (1024, 3584, 3584), (77, 1000, 4096), (640, 72, 200)]


@pytest.mark.parametrize("m,n,k", PAIR_SHAPES)
def test_gemm_pair_forward_and_bias(m, n, k):
    torch.manual_seed(0)
    a = (torch.randn(m, k, device=DEV) * 0.5).bfloat16()
    b = (torch.randn(n, k, device=DEV) * 0.5).bfloat16()
    bias = torch.randn(n, device=DEV).bfloat16()
    ref = a.float() @ b.float().t()
    _assert_close(G.gemm_pair(a, b), ref, k)
    _assert_close(G.gemm_pair(a, b, bias=bias), ref + bias.float(), k)
    G.check_status(DEV)


@pytest.mark.parametrize("m,n,k,splits", [(256, 512, 2048, 4), (200, 1000, 4096, 5), (256, 3584, 18944, 5),
                                          (130, 264, 1536, 3), (64, 256, 640, 16)])
def test_gemm_pair_split_reduction(m, n, k, splits):
    """Small-M form: the reduction cut into pieces (including pieces of unequal length and more pieces
    asked for than the planner would give), partial tiles added in a fixed order, optional bias."""
    torch.manual_seed(2)
    a = (torch.randn(m, k, device=DEV) * 0.5).bfloat16()
    b = (torch.randn(n, k, device=DEV) * 0.5).bfloat16()
    bias = torch.randn(n, device=DEV).bfloat16()
    ref = a.float() @ b.float().t()
    out1 = G.gemm_pair_splitk(a, b, splits)
    _assert_close(out1, ref, k)
    _assert_close(G.gemm_pair_splitk(a, b, splits, bias=bias), ref + bias.float(), k)
    assert torch.equal(out1, G.gemm_pair_splitk(a, b, splits))      # fixed summation order
    G.check_status(DEV)


def test_linear_fwd_routes_decode_shapes():
    """256-token decode shapes: wide outputs on the plain pair kernel, long reductions on the split
    form, the rest on the library; all three agree with the fp32 product."""
    torch.manual_seed(3)
    for n, k in [(37888 // 8, 3584), (3584, 18944), (4608, 3584)]:
        x = (torch.randn(256, k, device=DEV) * 0.5).bfloat16()
        w = (torch.randn(n, k, device=DEV) * 0.5).bfloat16()
        _assert_close(G.linear_fwd(x, w), x.float() @ w.float().t(), k)
    assert G.splitk_plan(256, 3584, 18944) >= 2 and G.splitk_plan(256, 4608, 3584) == 0
    G.check_status(DEV)


@pytest.mark.parametrize("m,n,k", PAIR_SHAPES)
def test_gemm_pair_data_and_weight_gradient_forms(m, n, k):
    """``dy @ w`` with ``w`` as an MN-major B operand, and ``dy.T @ x`` with both operands MN-major,
    stored and accumulated into fp32 / bf16 gradient buffers."""
    torch.manual_seed(1)
    dy = (torch.randn(m, k, device=DEV) * 0.5).bfloat16()         # [T, N_lin] : reduction over its columns
    w = (torch.randn(k, n, device=DEV) * 0.5).bfloat16()          # [N_lin, K_lin] read as stored
    _assert_close(G.gemm_pair(dy, w, b_mn=True), dy.float() @ w.float(), k)
    t = k                                                          # tokens are the reduction of the weight gradient
    t8 = (t + 7) // 8 * 8
    g_out = (torch.randn(t8, m // 8 * 8 or 8, device=DEV) * 0.5).bfloat16()
    x_in = (torch.randn(t8, n // 8 * 8 or 8, device=DEV) * 0.5).bfloat16()
    ref = g_out.float().t() @ x_in.float()
    _assert_close(G.gemm_pair(g_out, x_in, a_mn=True, b_mn=True), ref, t8)
    for dt in (torch.float32, torch.bfloat16):
        base = torch.randn(ref.shape, device=DEV).to(dt)
        grad = base.clone()
        mode = "acc_f32" if dt == torch.float32 else "acc_bf16"
        G.gemm_pair(g_out, x_in, a_mn=True, b_mn=True, out=grad, mode=mode)
        G.gemm_pair(g_out, x_in, a_mn=True, b_mn=True, out=grad, mode=mode)
        _assert_close(grad, base.float() + 2 * ref, 4 * t8)
    G.check_status(DEV)


@pytest.mark.parametrize("t,v,h", [(200, 1000, 256), (513, 5000, 896)])
def test_lmhead_stats_fused(t, v, h):
    torch.manual_seed(1)
    x = torch.randn(t, h, device=DEV).bfloat16()
    w = (0.05 * torch.randn(v, h, device=DEV)).bfloat16()
    y = torch.randint(0, v, (t,), device=DEV)
    stats, tiles = G.lmhead_stats(x, w, y, 1 / 0.7)
    G.check_status(DEV)
    logp = torch.empty(t, device=DEV)
    ent = torch.empty(t, device=DEV)
    lse = torch.empty(t, device=DEV)
    L = _lib.load()
    assert L.msrl_logprob_finish(ptr(stats), c_int(tiles), c_ll(t), ptr(logp), ptr(ent), ptr(lse), stream()) == 0
    z = (x.float() @ w.float().t()).bfloat16().float() / 0.7
    ls = torch.log_softmax(z, -1)
    ref_lp = ls.gather(-1, y[:, None])[:, 0]
    ref_ent = -(ls.exp() * ls).sum(-1)
    assert (logp - ref_lp).abs().max() < 3e-2, (logp - ref_lp).abs().max()
    assert (ent - ref_ent).abs().max() < 3e-2, (ent - ref_ent).abs().max()


@pytest.mark.parametrize("ml,k,n", [(128, 256, 256), (384, 512, 776), (1024, 1024, 1536)])
def test_fused_comm_gemm_single_rank(ml, k, n):
    """World size 1 exercises the comm warps, counters and tile order of both fused variants
    (self-gather, push to the own staging area) without a second GPU."""
    from mindspeed_rl_b200.parallel.fused_tp import FusedTP
    from mindspeed_rl_b200.parallel.symm import SymmetricArena

    torch.manual_seed(3)
    arena = SymmetricArena(8 * ml * max(k, n) * 2 + (8 << 20))
    try:
        f = FusedTP(arena, [0], ml, k, n)
        for call in range(3):
            x = (torch.randn(ml, k, device=DEV) * 0.5).bfloat16()
            w = (torch.randn(n, k, device=DEV) * 0.5).bfloat16()
            assert f.fits_ag(x, w) and f.fits_rs(x, w)
            y, xg = f.ag_gemm(x, w)
            G.check_status(x.device)
            assert torch.equal(xg, x)
            ref = x.float() @ w.float().t()
            assert bool(((y.float() - ref).abs() <= 2e-2 * ref.abs() + 0.25).all()), call
            out = f.gemm_rs(x, w)
            G.check_status(x.device)
            assert bool(((out.float() - ref).abs() <= 2e-2 * ref.abs() + 0.25).all()), call
        arena.check()
    finally:
        arena.close()


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("nh,nkv,interleaved", [(4, 2, True), (7, 1, False)])
def test_flash_attention_fwd_tcgen05(nh, nkv, interleaved, causal, monkeypatch):
    """tcgen05 forward attention against the fp32 oracle and the mma.sync kernel: ragged packed
    sequences that end inside a key tile, one longer than several tiles, a single token."""
    from mindspeed_rl_b200 import ops
    from mindspeed_rl_b200.ops.layouts import QKVLayout
    torch.manual_seed(11)
    lay = QKVLayout(nh, nkv, 128, interleaved)
    lens = [1, 129, 640, 77, 1000, 256]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    t = int(cu[-1])
    qkv = (0.7 * torch.randn(t, lay.width, device="cuda")).bfloat16()
    monkeypatch.setenv("MSRL_ATTN_TCGEN05", "1")
    out, lse = ops.attn_varlen_fwd(qkv, lay, cu.cuda(), max(lens), causal=causal)
    G.check_status(torch.device("cuda", torch.cuda.current_device()), "tcgen05 attention")
    monkeypatch.setenv("MSRL_ATTN_TCGEN05", "0")
    out_m, lse_m = ops.attn_varlen_fwd(qkv, lay, cu.cuda(), max(lens), causal=causal)
    out_r, lse_r = ops.attn_varlen_fwd(qkv.cpu(), lay, cu, max(lens), causal=causal)
    torch.testing.assert_close(out.float().cpu(), out_r.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(lse.cpu(), lse_r, rtol=1e-2, atol=2e-2)
    torch.testing.assert_close(out.float(), out_m.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(lse, lse_m, rtol=1e-2, atol=2e-2)


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("nh,nkv,interleaved", [(4, 2, True), (7, 1, False)])
def test_flash_attention_bwd_tcgen05(nh, nkv, interleaved, causal, monkeypatch):
    """tcgen05 backward (dQ kernel, dK/dV kernel, delta) against autograd through the fp32
    formulation and against the mma.sync kernels."""
    from mindspeed_rl_b200 import ops
    from mindspeed_rl_b200.ops.layouts import QKVLayout
    torch.manual_seed(12)
    lay = QKVLayout(nh, nkv, 128, interleaved)
    lens = [1, 129, 640, 77, 1000, 256]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    t = int(cu[-1])
    qkv = (0.7 * torch.randn(t, lay.width, device="cuda")).bfloat16()
    dout = (0.5 * torch.randn(t, nh * 128, device="cuda")).bfloat16()
    monkeypatch.setenv("MSRL_ATTN_TCGEN05", "1")
    out, lse = ops.attn_varlen_fwd(qkv, lay, cu.cuda(), max(lens), causal=causal)
    dqkv = ops.attn_varlen_bwd(dout, qkv, out, lse, lay, cu.cuda(), max(lens), causal=causal)
    G.check_status(torch.device("cuda", torch.cuda.current_device()), "tcgen05 attention")
    monkeypatch.setenv("MSRL_ATTN_TCGEN05", "0")
    dqkv_m = ops.attn_varlen_bwd(dout, qkv, out, lse, lay, cu.cuda(), max(lens), causal=causal)
    out_r, lse_r = ops.attn_varlen_fwd(qkv.cpu(), lay, cu, max(lens), causal=causal)
    dqkv_r = ops.attn_varlen_bwd(dout.cpu(), qkv.cpu(), out_r, lse_r, lay, cu, max(lens), causal=causal)
    torch.testing.assert_close(dqkv.float().cpu(), dqkv_r.float(), rtol=3e-2, atol=5e-2)
    torch.testing.assert_close(dqkv.float(), dqkv_m.float(), rtol=3e-2, atol=5e-2)


@pytest.mark.parametrize("causal", [False, True])
def test_block_attention_with_separate_kv(causal):
    """The block primitives of ring attention (queries against a separate K/V block, log-sum-exp of the
    whole row given to the backward) against the fp32 formulation: ragged query and key lengths,
    non-causal and bottom-right causal."""
    from mindspeed_rl_b200 import ops
    torch.manual_seed(21)
    nh, nkv, hd = 6, 2, 128
    ql, kl = [130, 64, 500], [257, 64, 900]
    cu_q = torch.tensor([0] + list(torch.tensor(ql).cumsum(0)), dtype=torch.int32)
    cu_k = torch.tensor([0] + list(torch.tensor(kl).cumsum(0)), dtype=torch.int32)
    tq, tk = int(cu_q[-1]), int(cu_k[-1])
    q = (0.7 * torch.randn(tq, nh, hd, device="cuda")).bfloat16()
    k = (0.7 * torch.randn(tk, nkv, hd, device="cuda")).bfloat16()
    v = (0.7 * torch.randn(tk, nkv, hd, device="cuda")).bfloat16()
    do = (0.5 * torch.randn(tq, nh * hd, device="cuda")).bfloat16()
    out, lse = ops.attn_kv_fwd(q, k, v, cu_q.cuda(), cu_k.cuda(), max(ql), causal)
    dq, dk, dv = ops.attn_kv_bwd(do, q, k, v, out, lse, cu_q.cuda(), cu_k.cuda(), max(ql), max(kl), causal)
    G.check_status(torch.device("cuda", torch.cuda.current_device()), "block attention")
    out_r, lse_r = ops.attn_kv_fwd(q.cpu().float(), k.cpu().float(), v.cpu().float(), cu_q, cu_k, max(ql), causal)
    dq_r, dk_r, dv_r = ops.attn_kv_bwd(do.cpu().float(), q.cpu().float(), k.cpu().float(), v.cpu().float(), out_r, lse_r,
                                       cu_q, cu_k, max(ql), max(kl), causal)
    torch.testing.assert_close(out.float().cpu(), out_r, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(lse.cpu(), lse_r, rtol=1e-2, atol=2e-2)
    for a, b in ((dq, dq_r), (dk, dk_r), (dv, dv_r)):
        torch.testing.assert_close(a.float().cpu(), b, rtol=3e-2, atol=5e-2)
