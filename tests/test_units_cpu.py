"""Unit tests with hand-computed expectations: masked statistics, KL estimators, advantages,
policy / value / DPO losses, padding helpers, sequence-length balancing, the experience store,
verifiers, the indexed dataset format, templates and the expert load balancer."""
import math

import numpy as np
import pytest
import torch

from mindspeed_rl_b200 import ops
from mindspeed_rl_b200.utils import torch_functional as F
from mindspeed_rl_b200.utils.compute import compute_kl_penalty
from mindspeed_rl_b200.utils.pad_process import (pad_rows, padding_dict_to_tensor_dict,
                                                 remove_padding_tensor_dict_to_dict, truncate_rows)
from mindspeed_rl_b200.utils.seqlen_balancing import (balanced_bin_packing, get_reverse_idx,
                                                      get_seqlen_balanced_partitions, rearrange_micro_batches)


# ---- masked statistics / KL ---------------------------------------------------------------------------------
def test_masked_statistics():
    v = torch.tensor([[1.0, 2.0, 3.0, 100.0], [4.0, 6.0, -50.0, -50.0]])
    m = torch.tensor([[1.0, 1.0, 1.0, 0.0], [1.0, 1.0, 0.0, 0.0]])
    assert float(F.masked_sum(v, m)) == 16.0
    assert float(F.masked_mean(v, m)) == pytest.approx(3.2)
    assert torch.allclose(F.masked_mean(v, m, axis=-1), torch.tensor([2.0, 5.0]))
    vals = torch.tensor([1.0, 2.0, 3.0, 4.0, 6.0])
    assert float(F.masked_var(v, m)) == pytest.approx(float(vals.var(unbiased=True)))
    w = F.masked_whiten(v, m)
    assert float(F.masked_mean(w, m)) == pytest.approx(0.0, abs=1e-6)
    assert torch.equal(F.clip_by_value(torch.tensor([-2.0, 0.5, 9.0]), torch.tensor(-1.0), torch.tensor(1.0)),
                       torch.tensor([-1.0, 0.5, 1.0]))
    assert torch.equal(F.sequence_mask(torch.tensor([1, 3]), 4), torch.tensor([[1.0, 0, 0, 0], [1, 1, 1, 0]]))


def test_kl_estimators():
    lp, ref = torch.tensor([-1.0, -2.0, -0.5]), torch.tensor([-1.5, -1.0, -0.5])
    assert torch.allclose(compute_kl_penalty(lp, ref, "kl"), torch.tensor([0.5, -1.0, 0.0]))
    assert torch.allclose(compute_kl_penalty(lp, ref, "abs"), torch.tensor([0.5, 1.0, 0.0]))
    assert torch.allclose(compute_kl_penalty(lp, ref, "mse"), torch.tensor([0.125, 0.5, 0.0]))
    k = ref - lp
    assert torch.allclose(compute_kl_penalty(lp, ref, "low_var_kl"), torch.exp(k) - k - 1)
    big = compute_kl_penalty(torch.tensor([-100.0]), torch.tensor([0.0]), "low_var_kl")
    assert float(big) == 10.0                               # exp(20) - 21 clamps to 10
    with pytest.raises(NotImplementedError):
        compute_kl_penalty(lp, ref, "nope")


# ---- advantages and losses --------------------------------------------------------------------------------------
def test_group_norm_advantage_and_gae():
    scores = torch.tensor([1.0, 0.0, 0.0, 1.0, 1.0, 1.0])          # two prompts x three samples
    mask = torch.tensor([[1.0, 1, 0], [1, 1, 1], [1, 0, 0], [1, 1, 1], [1, 1, 0], [1, 0, 0]])
    adv = ops.group_norm_advantage(scores, mask, 3)
    g0 = scores[:3]
    want0 = (g0 - g0.mean()) / (g0.std(unbiased=True) + 1e-6)
    assert torch.allclose(adv[:3], want0.unsqueeze(1) * mask[:3], atol=1e-5)
    assert torch.equal(adv[3:], torch.zeros(3, 3))                 # identical scores -> zero advantage
    # GAE, gamma = lam = 1, no whitening: advantage_t = sum_{s>=t} r_s - v_t
    r = torch.tensor([[0.0, 0.0, 1.0]])
    v = torch.tensor([[0.2, 0.4, 0.6]])
    a, ret = ops.gae(r, v, torch.ones(1, 3), 1.0, 1.0, whiten=False)
    assert torch.allclose(a, torch.tensor([[0.8, 0.6, 0.4]]), atol=1e-6)
    assert torch.allclose(ret, a + v, atol=1e-6)
    a2, _ = ops.gae(r, v, torch.ones(1, 3), 0.5, 0.0, whiten=False)  # lam = 0: one-step TD errors
    assert torch.allclose(a2, torch.tensor([[0.0, -0.1, 0.4]]), atol=1e-6)


def test_policy_and_value_loss_against_formulas():
    torch.manual_seed(0)
    b, l = 3, 5
    logp = (torch.randn(b, l) * 0.3).requires_grad_(True)
    old, ref, adv = logp.detach() + torch.randn(b, l) * 0.2, torch.randn(b, l) * 0.3, torch.randn(b, l)
    mask = (torch.rand(b, l) > 0.3).float()
    mask[:, 0] = 1
    lo, hi, beta = 0.2, 0.28, 0.05
    ratio = torch.exp(logp - old)
    pg = torch.max(-adv * ratio, -adv * ratio.clamp(1 - lo, 1 + hi))
    k = (ref - logp).clamp(-20, 20)
    kl = (torch.exp(k) - k - 1).clamp(-10, 10)
    want = (pg * mask).sum() / mask.sum() + beta * (kl * mask).sum() / mask.sum()
    (g_want,) = torch.autograd.grad(want, logp)
    grad, stats = ops.policy_loss_fwd_bwd(logp.detach(), old, ref, adv, mask, lo, hi, beta, "low_var_kl", True)
    assert torch.allclose(grad, g_want, atol=1e-6)
    assert float(stats["pg_loss"]) == pytest.approx(float((pg * mask).sum() / mask.sum()), abs=1e-6)
    assert float(stats["kl_loss"]) == pytest.approx(float((kl * mask).sum() / mask.sum()), abs=1e-6)
    # clipped value loss
    vp = torch.randn(b, l, requires_grad=True)
    vals, rets, clip = vp.detach() + 0.3 * torch.randn(b, l), torch.randn(b, l), 0.2
    vclip = vals + (vp - vals).clamp(-clip, clip)
    vf = 0.5 * (torch.max((vp - rets) ** 2, (vclip - rets) ** 2) * mask).sum() / mask.sum()
    (gv_want,) = torch.autograd.grad(vf, vp)
    gv, vst = ops.value_loss_fwd_bwd(vp.detach(), vals, rets, mask, clip)
    assert torch.allclose(gv, gv_want, atol=1e-6) and float(vst["vf_loss"]) == pytest.approx(float(vf), abs=1e-6)


def test_dpo_loss_values():
    from mindspeed_rl_b200.trainer.dpo_trainer import dpo_loss
    pc, pr, rc, rr = torch.tensor([-1.0]), torch.tensor([-3.0]), torch.tensor([-2.0]), torch.tensor([-2.5])
    margin = (pc - pr) - (rc - rr)                                   # 1.5
    loss, cr, rj = dpo_loss(pc, pr, rc, rr, beta=0.1)
    assert float(loss) == pytest.approx(-math.log(1 / (1 + math.exp(-0.15))), abs=1e-6)
    assert float(cr) == pytest.approx(0.1) and float(rj) == pytest.approx(-0.05)
    assert float(dpo_loss(pc, pr, rc, rr, 0.1, "hinge")[0]) == pytest.approx(1 - 0.15)
    assert float(dpo_loss(pc, pr, rc, rr, 0.1, "ipo")[0]) == pytest.approx((float(margin) - 5.0) ** 2)


# ---- padding / balancing ---------------------------------------------------------------------------------------------
def test_padding_round_trip():
    rows = {"a": [torch.tensor([1, 2, 3]), torch.tensor([4])], "b": [torch.tensor([0.5]), torch.tensor([1.5, 2.5])]}
    packed = padding_dict_to_tensor_dict(rows)
    assert packed["a"].shape == (2, 3) and "original_length" in packed
    back = remove_padding_tensor_dict_to_dict(packed)
    assert all(torch.equal(x, y) for k in rows for x, y in zip(rows[k], back[k]))
    assert pad_rows([torch.tensor([1]), torch.tensor([1, 2, 3])], 9, multiple=4).tolist() == [[1, 9, 9, 9], [1, 2, 3, 9]]
    t = truncate_rows(torch.tensor([[1, 2, 3, 0], [4, 0, 0, 0]]), torch.tensor([3, 1]))
    assert [x.tolist() for x in t] == [[1, 2, 3], [4]]


def test_seqlen_balancing():
    lens = [10, 90, 20, 80, 30, 70, 40, 60]
    parts = get_seqlen_balanced_partitions(lens, 4, equal_size=True)
    assert sorted(i for p in parts for i in p) == list(range(8)) and all(len(p) == 2 for p in parts)
    assert {sum(lens[i] for i in p) for p in parts} == {100}
    bins = balanced_bin_packing([50, 40, 30, 30, 20, 10, 10], 100)
    assert all(sum([50, 40, 30, 30, 20, 10, 10][i] for i in b) <= 100 for b in bins) and len(bins) == 2
    mbs = rearrange_micro_batches([60, 50, 40, 30, 20], 100, None, None)
    assert all(sum([60, 50, 40, 30, 20][i] for i in m) <= 100 for m in mbs)
    assert get_reverse_idx([2, 0, 1]) == [1, 2, 0]


# ---- experience store ----------------------------------------------------------------------------------------------------
def test_transfer_dock_semantics():
    from mindspeed_rl_b200.data.transfer_dock import GRPOTransferDock, put_prompts_experience
    td = GRPOTransferDock(2, 2)
    data, idx = put_prompts_experience({"prompts": [torch.arange(3), torch.arange(5)]}, 2)
    assert idx == [0, 1, 2, 3] and [int(x) for x in data["prompt_length"]] == [3, 3, 5, 5]
    td.put_experience(data, idx)
    assert not td.all_consumed("actor_rollout")
    batch, got = td.get_experience("actor_rollout", ["prompts", "prompt_length"], 2, get_n_samples=True)
    assert got in ([0, 1], [2, 3]) and batch["prompts"].shape[0] == 2          # whole groups only
    _, rest = td.get_experience("actor_rollout", ["prompts"], 2, get_n_samples=True)
    assert sorted(got + rest) == [0, 1, 2, 3] and td.all_consumed("actor_rollout")
    assert td.get_experience("actor_train", ["responses"], 2) == (None, None)     # not produced yet
    td.put_experience({"responses": [torch.tensor([7, 8]), torch.tensor([9])]}, [0, 1])
    b2, i2 = td.get_experience("actor_train", ["responses"], 2, get_n_samples=True)
    assert i2 == [0, 1] and b2["responses"].tolist() == [[7, 8], [9, 0]]
    with pytest.raises(ValueError):
        td.get_experience("nobody", ["prompts"], 2)
    with pytest.raises(ValueError):
        td.put_experience({"unknown_column": [torch.ones(1)]}, [0])
    td.update_metrics("x", value=[1.0, 3.0], cumulate=True)
    td.clear()
    assert td.get_experience("actor_rollout", ["prompts"], 2) == (None, None)


# ---- verifiers ------------------------------------------------------------------------------------------------------------
def test_rule_verifiers():
    from mindspeed_rl_b200.rewards import math_verifiers as mv
    from mindspeed_rl_b200.rewards.registry import known_verifiers, overlong_penalty
    good = "<think>\n2+2=4\n</think>\n<answer>\n\\boxed{4}\n</answer>"
    assert mv.accuracy_reward([good, "<answer>\\boxed{5}</answer>", "no box at all"], ["4", "4", "4"]) == [1.0, -0.5, -1.0]
    assert mv.format_reward([good, "no tags"])[0] == 1.0 and mv.format_reward([good, "no tags"])[1] == 0.0
    assert mv.math_17k_accuracy_reward(["so the answer is \\boxed{\\frac{1}{2}}"], ["1/2"])[0] == 1.0
    assert mv.dapo_accuracy_reward(["Answer: 7"], ["7"])[0] in (1.0, -1.0)
    assert {"acc", "format", "math_17k_acc", "acc_for_dapo", "acc_for_ppo", "contains_token_7"} <= set(known_verifiers())
    assert overlong_penalty(100, 200, 50, 1.0) == 0.0
    assert overlong_penalty(175, 200, 50, 1.0) == pytest.approx(-0.5)
    assert overlong_penalty(260, 200, 50, 2.0) == pytest.approx(-2.0)


# ---- dataset format / templates ---------------------------------------------------------------------------------------------
def test_indexed_dataset_round_trip(tmp_path):
    from mindspeed_rl_b200.datasets.indexed_dataset import (IndexedDataset, IndexedDatasetBuilder, get_bin_path,
                                                            get_idx_path)
    prefix = str(tmp_path / "toy_packed_input_ids_document")
    docs = [[1, 2, 3], [4], [5, 6, 7, 8, 9]]
    b = IndexedDatasetBuilder(get_bin_path(prefix), dtype=np.int32)
    for d in docs:
        b.add_item(torch.tensor(d))
        b.end_document()
    b.finalize(get_idx_path(prefix))
    assert open(get_idx_path(prefix), "rb").read(9) == b"MMIDIDX\x00\x00"
    ds = IndexedDataset(prefix)
    assert len(ds) == 3 and [ds[i].tolist() for i in range(3)] == docs
    assert ds.get(2, offset=1, length=3).tolist() == [6, 7, 8]


def test_chat_template_renders_turns():
    import os
    from mindspeed_rl_b200.datasets.templates import get_model_template
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "configs", "model", "templates.json")
    tpl = get_model_template("qwen", path)

    class Tok:
        eos_token, eos_token_id = "<|im_end|>", 2
        def encode(self, text, add_special_tokens=False):
            return [ord(c) for c in text]
        def convert_tokens_to_ids(self, t):
            return 2
    pairs = tpl.encode_multiturn(Tok(), [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "yo"}])
    text = "".join(chr(c) for ids in pairs[0] for c in ids)
    assert "<|im_start|>user\nhi<|im_end|>" in text and text.endswith("yo<|im_end|>\n") or "yo" in text


# ---- expert load balancer ------------------------------------------------------------------------------------------------------
def test_eplb_invariants():
    from mindspeed_rl_b200.rollout.eplb import expert_map_from_counts, rebalance_experts
    torch.manual_seed(0)
    w = torch.randint(1, 100, (2, 16)).float()
    w[:, 3] = 1000                                                   # one hot expert
    phy2log, log2phy, logcnt = rebalance_experts(w, 24, num_groups=4, num_nodes=2, num_gpus=8)
    assert phy2log.shape == (2, 24) and int(logcnt.sum()) == 48 and int(logcnt.min()) >= 1
    assert int(logcnt[0, 3]) == int(logcnt[0].max()) > 1             # the hot expert got replicas
    for l in range(2):
        for e in range(16):
            slots = log2phy[l, e][log2phy[l, e] >= 0]
            assert len(slots) == int(logcnt[l, e]) and (phy2log[l, slots] == e).all()
    m = expert_map_from_counts(w, num_gpus=8, num_redundancy_per_gpu=1)
    assert m["moe_layer_count"] == 2
    for layer in m["layer_list"]:
        hosted = [e for d in layer["device_list"] for e in d["device_expert"]]
        assert set(hosted) == set(range(16)) and all(len(set(d["device_expert"])) == 3 for d in layer["device_list"])


def test_reuse_fp32_param_split_is_exact_and_tracks_fp32_master():
    """bf16 parameter + int16 residual reproduce every fp32 bit pattern; an optimizer that keeps
    only the residual follows the one with fp32 master weights."""
    from mindspeed_rl_b200.optim.distributed_optimizer import DistributedOptimizer
    from mindspeed_rl_b200.parallel.ddp import DistributedDataParallel
    torch.manual_seed(0)
    x = torch.randn(100000) * torch.logspace(-6, 3, 100000)
    x[:4] = torch.tensor([0.0, -0.0, 1.00390625, -3.0])          # includes an exact tie (1 + 2^-8)
    p16 = torch.empty(100000, dtype=torch.bfloat16)
    lo = torch.empty(100000, dtype=torch.int16)
    DistributedOptimizer.split_master(x, p16, lo)
    assert torch.equal(DistributedOptimizer.compose_master(p16, lo), x)
    assert (p16.float() - x).abs().max() <= (x.abs() * 2 ** -8).max()

    def make(reuse):
        torch.manual_seed(1)
        lin = torch.nn.Linear(64, 64, bias=False).bfloat16()
        m = DistributedDataParallel(lin)
        return m, DistributedOptimizer(m.buffers, lr=1e-2, weight_decay=0.1, clip_grad=0.0, reuse_fp32_param=reuse)

    (ma, oa), (mb, ob) = make(False), make(True)
    assert ob.reuse_fp32_param and "master_lo" in ob.state[0]
    for step in range(5):
        g = torch.Generator().manual_seed(step)
        for m in (ma, mb):
            m.buffers[0].grad_data.copy_(torch.randn(m.buffers[0].grad_data.shape, generator=g.manual_seed(step)))
        oa.step()
        ob.step()
    wa, wb = ma.buffers[0].param_data.float(), mb.buffers[0].param_data.float()
    assert (wa - wb).abs().max() <= 2 ** -7 * wa.abs().max()      # at most one bf16 ulp apart (tie rounding)
    full = ob.state_dict()["shards"][0]["master"]
    torch.testing.assert_close(full, oa.state[0]["master"], rtol=1e-6, atol=1e-7)


def test_pack_tokens_and_unpack_response_reference_path():
    """The packing op against the definition: ids / shifted labels / restarting positions of every
    block, zeros in block padding; response rows start at the position that predicts the first
    response token."""
    import torch
    from mindspeed_rl_b200.ops.packing import pack_tokens, unpack_response
    g = torch.Generator().manual_seed(0)
    p_len = torch.tensor([3, 5, 1], dtype=torch.int32)
    r_len = torch.tensor([4, 2, 6], dtype=torch.int32)
    s = 10
    ids2d = torch.randint(1, 100, (3, s), generator=g)
    lens = (p_len + r_len).long()
    padded = (lens + 3) // 4 * 4
    cu = torch.zeros(4, dtype=torch.int32)
    cu[1:] = torch.cumsum(padded, 0)
    total = int(cu[-1])
    ids, labels, pos = pack_tokens(ids2d, p_len, r_len, cu, total)
    for b in range(3):
        lo, n = int(cu[b]), int(lens[b])
        assert ids[lo:lo + n].tolist() == ids2d[b, :n].tolist()
        assert labels[lo:lo + n - 1].tolist() == ids2d[b, 1:n].tolist() and int(labels[lo + n - 1]) == 0
        assert ids[lo + n:int(cu[b + 1])].sum() == 0 and labels[lo + n:int(cu[b + 1])].sum() == 0
        assert pos[lo:int(cu[b + 1])].tolist() == list(range(int(padded[b])))
    src = torch.arange(total, dtype=torch.float32) + 1
    out = unpack_response(src, cu, p_len, r_len, 6)
    for b in range(3):
        start = int(cu[b]) + int(p_len[b]) - 1
        want = [float(src[start + j]) if j < int(r_len[b]) else 0.0 for j in range(6)]
        assert out[b].tolist() == want


def test_flat_buffers_release_and_restore_plain_allocations():
    """Without peer-mapped memory the offloaders free plain allocations: gradients come back zeroed,
    parameters come back from the pinned-host twin, and the parameters point at the new storage."""
    from mindspeed_rl_b200.parallel.ddp import DistributedDataParallel
    from mindspeed_rl_b200.reshard.sharding_manager import GradBufferOffloader, ParamOffloader

    torch.manual_seed(0)
    net = torch.nn.Linear(16, 8)
    ddp = DistributedDataParallel(net, None, 1, releasable_params=True, releasable_grads=True)
    buf = ddp.buffers[0]
    assert buf.arena is None and buf._own == {"param": False, "grad": False}
    want = buf.param_data.clone()
    net.weight.main_grad.fill_(3.0)
    grads, params = GradBufferOffloader(ddp), ParamOffloader(ddp)
    grads.release()
    params.offload()
    assert buf.grad_data.numel() == 0 and buf.param_data.numel() == 0 and net.weight.main_grad is None
    params.onload()
    grads.restore()
    assert torch.equal(buf.param_data, want) and float(buf.grad_data.abs().sum()) == 0.0
    assert net.weight.data_ptr() == buf.param_data.data_ptr() and net.weight.main_grad.shape == net.weight.shape
    grads.restore()        # idempotent
    params.onload()


def test_canary_guard_passthrough_on_cpu(monkeypatch):
    """The debug allocator is a plain ``torch.empty`` for host tensors and when the mode is off."""
    from mindspeed_rl_b200.ops import guard

    monkeypatch.setenv("MSRL_DEBUG_CANARY", "1")
    t = guard.empty(3, 5, dtype=torch.float32, device="cpu")
    assert t.shape == (3, 5) and guard.check("cpu") == 0
    assert guard.empty_like(t).shape == (3, 5) and guard.empty((2, 2), dtype=torch.int32).dtype == torch.int32


def test_kv_cache_cap_follows_the_engine_limits():
    """The KV cache is capped at what the configured sequences can occupy, unless a prefix cache can use more."""
    from types import SimpleNamespace

    from mindspeed_rl_b200.reshard.sharding_manager import ShardingManager

    eng = SimpleNamespace(device=torch.device("cpu"), max_model_len=3072, block_size=16, max_num_seqs=256,
                          enable_prefix_caching=False)
    sm = ShardingManager(torch.nn.Linear(2, 2), eng)
    assert sm._kv_block_cap() == 256 * (3072 // 16 + 1)
    eng.enable_prefix_caching = True
    assert sm._kv_block_cap() is None
    assert sm._release_needed()                      # no device memory to reason about on the CPU: release as asked
    assert sm._kv_blocks() == 256
