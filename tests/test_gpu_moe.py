"""MoE kernels (plan, permute, combine, slot-dot, grouped tcgen05 GEMM) against the PyTorch
formulation of the same ops."""
import pytest
import torch

from mindspeed_rl_b200.ops import gemm as G
from mindspeed_rl_b200.ops import moe as M

pytestmark = pytest.mark.gpu


def _cpu_plan(plan):
    return M.MoePlan(plan.counts.cpu(), plan.offsets.cpu(), plan.pos.cpu(), plan.tile_expert.cpu(), plan.max_rows,
                     plan.tokens, plan.k, plan.num_experts)


@pytest.mark.parametrize("t,k,e", [(1000, 8, 128), (37, 2, 4), (5000, 8, 16)])
def test_plan_matches_reference(t, k, e):
    torch.manual_seed(0)
    idx = torch.randint(0, e, (t, k), device="cuda")
    plan = M.moe_plan(idx, e)
    ref = M.moe_plan(idx.cpu(), e)
    assert plan.counts.cpu().tolist() == ref.counts.tolist()
    assert plan.offsets.cpu().tolist() == ref.offsets.tolist()
    assert plan.pos.cpu().tolist() == ref.pos.tolist()
    assert plan.tile_expert.cpu().tolist() == ref.tile_expert.tolist()


@pytest.mark.parametrize("t,k,e,h,f", [(777, 8, 16, 2048, 768), (130, 2, 4, 256, 128)])
def test_moe_layer_kernels(t, k, e, h, f):
    torch.manual_seed(1)
    dev = "cuda"
    x = torch.randn(t, h, device=dev).bfloat16()
    idx = torch.stack([torch.randperm(e, device=dev)[:k] for _ in range(t)])
    p = torch.rand(t, k, device=dev)
    w1 = (torch.randn(h, e, 2 * f, device=dev) * 0.05).bfloat16()
    w2 = (torch.randn(e, f, h, device=dev) * 0.05).bfloat16()
    plan = M.moe_plan(idx, e)
    cplan = _cpu_plan(plan)
    xp = M.moe_permute(x, plan)
    xp_r = M.moe_permute(x.cpu(), cplan)
    used = int(plan.offsets[-1])
    assert torch.equal(xp[:used].cpu(), xp_r[:used])
    # forward: MN-major operands
    gu = M.grouped_gemm(xp, plan, w1.view(h, e * 2 * f), True, 2 * f, 0, 2 * f)
    gu_r = M.grouped_gemm(xp_r.float(), cplan, w1.cpu().float().view(h, e * 2 * f), True, 2 * f, 0, 2 * f)
    torch.testing.assert_close(gu[:used].float().cpu(), gu_r[:used], rtol=2e-2, atol=2e-2)
    act = (torch.nn.functional.silu(gu[:, :f].float()) * gu[:, f:].float()).bfloat16()
    act[used:] = 0
    y = M.grouped_gemm(act, plan, w2.view(e * f, h), True, 0, f, h)
    y_r = M.grouped_gemm(act.cpu().float(), cplan, w2.cpu().float().view(e * f, h), True, 0, f, h)
    torch.testing.assert_close(y[:used].float().cpu(), y_r[:used], rtol=2e-2, atol=2e-2)
    out = M.moe_combine(y, plan, p)
    out_r = M.moe_combine(y.cpu().float(), cplan, p.cpu())
    torch.testing.assert_close(out.float().cpu(), out_r, rtol=2e-2, atol=2e-2)
    # backward: scaled scatter, K-major operands, slot dot
    dout = torch.randn(t, h, device=dev).bfloat16()
    dy = M.moe_permute(dout, plan, p)
    dy_r = M.moe_permute(dout.cpu().float(), cplan, p.cpu())
    torch.testing.assert_close(dy[:used].float().cpu(), dy_r[:used], rtol=1e-2, atol=1e-2)
    dact = M.grouped_gemm(dy, plan, w2.view(e * f, h), False, 0, f, f)
    dact_r = M.grouped_gemm(dy.cpu().float(), cplan, w2.cpu().float().view(e * f, h), False, 0, f, f)
    torch.testing.assert_close(dact[:used].float().cpu(), dact_r[:used], rtol=2e-2, atol=2e-2)
    real = torch.zeros(plan.max_rows, 1, device=dev)
    real[plan.pos.long()] = 1                       # pad rows stay zero, as after a real backward
    dgu = (torch.randn(plan.max_rows, 2 * f, device=dev) * real).bfloat16()
    dxp = M.grouped_gemm(dgu, plan, w1.view(h, e * 2 * f), False, 2 * f, 0, h)
    dxp_r = M.grouped_gemm(dgu.cpu().float(), cplan, w1.cpu().float().view(h, e * 2 * f), False, 2 * f, 0, h)
    torch.testing.assert_close(dxp[:used].float().cpu(), dxp_r[:used], rtol=2e-2, atol=3e-2)
    dw = M.moe_slot_dot(dout, y, plan)
    dw_r = M.moe_slot_dot(dout.cpu().float(), y.cpu().float(), cplan)
    torch.testing.assert_close(dw.cpu(), dw_r, rtol=2e-2, atol=2e-2)
    G.check_status(torch.device("cuda", torch.cuda.current_device()), "grouped gemm")


def test_peer_memory_dispatch_overflow_falls_back():
    """A slab too small for the routing: with the fallback on, ``dispatch`` returns ``None`` and leaves the
    status word alone; with it off, the overflow is recorded for the stage-boundary check."""
    from mindspeed_rl_b200.parallel.moe_dispatch import P2PDispatcher
    from mindspeed_rl_b200.parallel.symm import SymmetricArena
    torch.manual_seed(4)
    t, k, e, h = 400, 4, 8, 128
    rows = 1024                                           # the routing below needs 8 experts x 256 padded rows
    arena = SymmetricArena(2 * P2PDispatcher.bytes_needed(1, e, h, rows) + (4 << 20))
    try:
        x = torch.randn(t, h, device="cuda").bfloat16()
        idx = torch.stack([torch.randperm(e, device="cuda")[:k] for _ in range(t)])
        soft = P2PDispatcher(arena, [0], e, h, rows, fallback=True)
        assert soft.dispatch(x, idx) is None and soft.overflows == 1
        arena.check()                                     # nothing recorded
        small = idx[:64]                                  # 8 experts x 128 padded rows fit exactly
        assert soft.dispatch(x[:64], small) is not None and soft.overflows == 1
        hard = P2PDispatcher(arena, [0], e, h, rows, fallback=False)
        hard.dispatch(x, idx)
        with pytest.raises(RuntimeError, match="overflow"):
            arena.check()
    finally:
        arena.close()


def test_peer_memory_dispatch_single_rank():
    """The peer-memory dispatch / combine kernels with a team of one rank (its own arena is the only
    "peer"): slab layout, rows, tile table and the weighted combine agree with the plan / permute /
    combine path."""
    from mindspeed_rl_b200.parallel.moe_dispatch import P2PDispatcher
    from mindspeed_rl_b200.parallel.symm import SymmetricArena
    torch.manual_seed(3)
    t, k, e, h = 517, 4, 8, 256
    rows = M.max_rows(t * k, e)
    arena = SymmetricArena(P2PDispatcher.bytes_needed(1, e, h, rows) + (4 << 20))
    try:
        disp = P2PDispatcher(arena, [0], e, h, rows)
        x = torch.randn(t, h, device="cuda").bfloat16()
        idx = torch.stack([torch.randperm(e, device="cuda")[:k] for _ in range(t)])
        w = torch.rand(t, k, device="cuda")
        route = disp.dispatch(x, idx)
        plan = M.moe_plan(idx, e)
        used = int(plan.offsets[-1])
        assert route.plan.counts.tolist() == plan.counts.tolist()
        assert route.plan.offsets.tolist() == plan.offsets.tolist()
        assert route.plan.tile_expert.tolist() == plan.tile_expert.tolist()
        assert route.slot_row.tolist() == plan.pos.tolist() and int(route.slot_rank.max()) == 0
        assert torch.equal(disp.slab[:used], M.moe_permute(x, plan)[:used])
        disp.out_slab.copy_(disp.slab * 2)                    # stand-in for the expert MLP
        out, kept = disp.combine(route, w, keep_rows=True)
        ref = M.moe_combine(M.moe_permute(x, plan) * 2, plan, w)
        torch.testing.assert_close(out.float(), ref.float(), rtol=1e-2, atol=1e-2)
        assert torch.equal(kept.view(t, k, h)[5, 2], disp.out_slab[int(plan.pos[5 * k + 2])])
        arena.check()
    finally:
        arena.close()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_grouped_weight_gradient_reads_segments_on_device(dtype):
    """Expert weight gradients in one launch per weight: every expert's ``a_e^T b_e`` is added into its block
    of the gradient view (blocks as column groups or as row groups), an expert without tokens is skipped, and
    the result matches the per-expert products."""
    torch.manual_seed(6)
    t, k, e, h, f = 900, 2, 6, 256, 192
    idx = torch.stack([torch.randperm(e - 1, device="cuda")[:k] + 1 for _ in range(t)])     # expert 0 gets nothing
    plan = M.moe_plan(idx, e)
    assert int(plan.counts[0]) == 0
    x = torch.randn(t, h, device="cuda").bfloat16()
    xp = M.moe_permute(x, plan)                                   # pad rows are zero
    dgu = torch.randn(plan.max_rows, 2 * f, device="cuda").bfloat16()
    act = torch.randn(plan.max_rows, f, device="cuda").bfloat16()
    dy = M.moe_permute(torch.randn(t, h, device="cuda").bfloat16(), plan)
    g1 = torch.randn(h, e, 2 * f, device="cuda").to(dtype)        # blocks = column groups
    g2 = torch.randn(e, f, h, device="cuda").to(dtype)            # blocks = row groups
    want1, want2 = g1.float().clone(), g2.float().clone()
    counts, offsets = plan.counts.tolist(), plan.offsets.tolist()
    for j, n in enumerate(counts):
        r = slice(offsets[j], offsets[j] + n)
        want1[:, j] += xp[r].float().t() @ dgu[r].float()
        want2[j] += act[r].float().t() @ dy[r].float()
    assert M.grouped_wgrad_(g1, 2 * f, e * 2 * f, xp, dgu, plan)
    assert M.grouped_wgrad_(g2, f * h, h, act, dy, plan)
    G.check_status("cuda", "grouped wgrad")
    tol = 2e-2 if dtype == torch.bfloat16 else 2e-3
    for got, want in ((g1, want1), (g2, want2)):
        err = (got.float() - want).abs().max().item()
        assert err <= tol * want.abs().max().item() + 1e-2, (dtype, err, want.abs().max().item())


def test_rollout_moe_with_shared_experts_on_side_stream():
    """Rollout expert layer with shared experts: computed on a side stream beside the routed experts (also
    when the layer is replayed from a CUDA graph) and equal to the single-stream result and the fp32 formula."""
    import os

    from mindspeed_rl_b200.models.transformer_config import TransformerConfig
    from mindspeed_rl_b200.rollout.moe import MoEWeights

    torch.manual_seed(8)
    t, e, k, h, f, fs = 300, 8, 2, 256, 128, 384
    cfg = TransformerConfig(num_layers=1, hidden_size=h, ffn_hidden_size=fs, num_attention_heads=2, num_query_groups=2,
                            vocab_size=64,
                            num_experts=e, moe_router_topk=k, moe_ffn_hidden_size=f, norm_topk_prob=True)
    router = torch.randn(e, h, device="cuda")
    w1 = (0.05 * torch.randn(h, e, 2 * f, device="cuda")).bfloat16()
    w2 = (0.05 * torch.randn(e, f, h, device="cuda")).bfloat16()
    shared = ((0.05 * torch.randn(2 * fs, h, device="cuda")).bfloat16(), (0.05 * torch.randn(h, fs, device="cuda")).bfloat16())
    layer = MoEWeights(cfg, router, w1, w2, shared=shared)
    x = torch.randn(t, h, device="cuda").bfloat16()
    forked = layer.forward(x)
    os.environ["MSRL_MOE_SHARED_STREAM"] = "0"
    try:
        plain = layer.forward(x)
    finally:
        del os.environ["MSRL_MOE_SHARED_STREAM"]
    assert torch.equal(forked, plain)
    without = MoEWeights(cfg, router, w1, w2).forward(x)
    g, u = (x.float() @ shared[0].float().t()).chunk(2, -1)
    want = without.float() + (torch.nn.functional.silu(g) * u).bfloat16().float() @ shared[1].float().t()
    assert (forked.float() - want).abs().max().item() <= 3e-2 * want.abs().max().item() + 1e-2
    # replay from a graph: the fork and the join are captured as graph edges
    static_x = x.clone()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        layer.forward(static_x)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = layer.forward(static_x)
    static_x.copy_(torch.randn(t, h, device="cuda").bfloat16())
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, layer.forward(static_x))
    G.check_status("cuda", "rollout moe")
