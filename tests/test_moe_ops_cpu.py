"""MoE dispatch plan, permute / combine and grouped GEMM (PyTorch formulation) against a dense
per-expert loop; token conservation."""
import torch

from mindspeed_rl_b200.ops import moe as M


def _dense(x, top_idx, top_p, w1, w2):
    """x [T,H]; w1 [H,E,2F]; w2 [E,F,H] -> sum_k p * (swiglu(x w1_e) w2_e)"""
    t, h = x.shape
    out = torch.zeros(t, h)
    f = w2.shape[1]
    for i in range(t):
        for j in range(top_idx.shape[1]):
            e = int(top_idx[i, j])
            gu = x[i].float() @ w1[:, e].float()
            act = torch.nn.functional.silu(gu[:f]) * gu[f:]
            out[i] += float(top_p[i, j]) * (act @ w2[e].float())
    return out


def test_plan_is_stable_and_conserves_tokens():
    torch.manual_seed(0)
    t, k, e = 300, 2, 7
    idx = torch.randint(0, e, (t, k))
    plan = M.moe_plan(idx, e)
    assert plan.counts.tolist() == torch.bincount(idx.reshape(-1), minlength=e).tolist()
    assert all(int(o) % M.PAD == 0 for o in plan.offsets.tolist())
    pos = plan.pos.long()
    assert pos.unique().numel() == t * k                      # no two slots share a row
    flat = idx.reshape(-1)
    for ex in range(e):
        rows = pos[flat == ex]
        lo = int(plan.offsets[ex])
        assert rows.tolist() == list(range(lo, lo + rows.numel()))   # in slot order, from the segment start
        assert (plan.tile_expert[lo // M.PAD:int(plan.offsets[ex + 1]) // M.PAD] == ex).all()
    assert (plan.tile_expert[int(plan.offsets[e]) // M.PAD:] == -1).all()


def test_permute_grouped_gemm_combine_matches_dense_loop():
    torch.manual_seed(1)
    t, k, e, h, f = 50, 2, 4, 64, 64
    x = torch.randn(t, h)
    idx = torch.stack([torch.randperm(e)[:k] for _ in range(t)])
    p = torch.rand(t, k)
    w1 = torch.randn(h, e, 2 * f) * 0.1
    w2 = torch.randn(e, f, h) * 0.1
    plan = M.moe_plan(idx, e)
    xp = M.moe_permute(x, plan)
    gu = M.grouped_gemm(xp, plan, w1.view(h, e * 2 * f), True, 2 * f, 0, 2 * f)
    act = torch.nn.functional.silu(gu[:, :f]) * gu[:, f:]
    y = M.grouped_gemm(act, plan, w2.view(e * f, h), True, 0, f, h)
    out = M.moe_combine(y, plan, p)
    torch.testing.assert_close(out, _dense(x, idx, p, w1, w2), rtol=1e-4, atol=1e-4)
    # K-major form (data gradients): d act = dy w2_e^T
    dy = M.moe_permute(torch.randn(t, h), plan, p)
    dact = M.grouped_gemm(dy, plan, w2.view(e * f, h), False, 0, f, f)
    r = int(plan.pos[3])
    e3 = int(idx.reshape(-1)[3])
    torch.testing.assert_close(dact[r], dy[r] @ w2[e3].t(), rtol=1e-4, atol=1e-4)
    # slot_dot: gradient of the combine weights
    dout = torch.randn(t, h)
    dw = M.moe_slot_dot(dout, y, plan)
    torch.testing.assert_close(dw[5, 1], (dout[5] * y[int(plan.pos[5 * k + 1])]).sum(), rtol=1e-4, atol=1e-4)
