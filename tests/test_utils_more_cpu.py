"""Packing helpers, context-parallel slicing, vocabulary-parallel log-probabilities and the samplers,
each against a direct PyTorch formulation."""
import math
import os
from types import SimpleNamespace

import pytest
import torch
import torch.distributed as dist

from dist_utils import run_distributed
from mindspeed_rl_b200.utils import context_parallel as CP
from mindspeed_rl_b200.utils import compute as U
from mindspeed_rl_b200.utils.remove_padding import packed_layout, postprocess_packed_seqs, preprocess_packed_seqs


def _padded_batch(lens, s, seed=0):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(1, 100, (len(lens), s), generator=g)
    mask = (torch.arange(s).unsqueeze(0) < torch.tensor(lens).unsqueeze(1)).long()
    return ids * mask, mask


def test_pack_and_unpack_padded_batch():
    lens, s, align = [5, 9, 1, 12], 12, 4
    ids, mask = _padded_batch(lens, s)
    labels = ids + 1000
    p_ids, pos, p_lab, seqlens, cu = preprocess_packed_seqs(ids, labels, mask, align)
    assert seqlens.tolist() == lens and cu.tolist() == [0, 8, 20, 24, 36] and cu.dtype == torch.int32
    assert p_ids.shape == (1, 36) and pos.shape == (1, 36)
    for b, n in enumerate(lens):
        lo, hi = int(cu[b]), int(cu[b + 1])
        assert p_ids[0, lo:lo + n].tolist() == ids[b, :n].tolist()
        assert p_lab[0, lo:lo + n].tolist() == labels[b, :n].tolist()
        assert p_ids[0, lo + n:hi].abs().sum() == 0                      # alignment padding is zero
        assert pos[0, lo:hi].tolist() == list(range(hi - lo))          # positions restart per block
    padded, cu2 = packed_layout(torch.tensor(lens), align)
    assert padded.tolist() == [8, 12, 4, 12] and torch.equal(cu2, cu)
    # back to [B, S, F] with a trailing feature dim
    feat = torch.stack([p_ids[0].float(), p_ids[0].float() * 2], dim=-1).unsqueeze(0)
    back = postprocess_packed_seqs(feat, seqlens, cu, s)
    assert back.shape == (4, s, 2)
    assert torch.equal(back[..., 0].long(), ids) and torch.equal(back[..., 1].long(), 2 * ids)
    # dropping the prompt: row b starts at the position that predicts the first response token
    prompt = torch.tensor([2, 4, 1, 12])
    out = postprocess_packed_seqs(p_ids.float(), seqlens, cu, 6, prompt_length=prompt)
    for b, (n, p) in enumerate(zip(lens, prompt.tolist())):
        if p - 1 < n:
            want = ids[b, p - 1:n - 1].tolist()[:6]
        else:
            want = ids[b, :n].tolist()[:6]
        assert out[b, :len(want)].long().tolist() == want, b
        assert out[b, len(want):].abs().sum() == 0
    with pytest.raises(ValueError):
        preprocess_packed_seqs(ids, labels, mask[:, :-1], align)


def test_context_parallel_slices_and_restore():
    cfg = SimpleNamespace(context_parallel_size=2, context_parallel_algo=CP.RING, reset_attention_mask=False)
    x = torch.arange(16).reshape(1, 16)
    kept = []
    for r in range(2):
        out, idx = CP.get_batch_on_this_cp_rank(cfg, {"tokens": x, "attention_mask": None, "none": None}, cp_rank=r)
        kept.append(idx)
        assert out["tokens"].tolist() == [[*range(4 * r, 4 * r + 4), *range(16 - 4 * (r + 1), 16 - 4 * r)]]
        assert out["attention_mask"] is None
    perm = CP.restore_permutation(torch.cat(kept))
    assert torch.cat([x[:, i] for i in kept], dim=1)[:, perm].tolist() == x.tolist()
    # packed: the zig-zag applies to every block on its own
    cfg.reset_attention_mask = True
    cu = torch.tensor([0, 8, 24], dtype=torch.int32)
    x = torch.arange(24).reshape(1, 24)
    got = [CP.get_batch_on_this_cp_rank(cfg, {"tokens": x}, cu, cp_rank=r)[0]["tokens"][0].tolist() for r in range(2)]
    assert got[0] == [0, 1, 6, 7, 8, 9, 10, 11, 20, 21, 22, 23]
    assert got[1] == [2, 3, 4, 5, 12, 13, 14, 15, 16, 17, 18, 19]
    # all-to-all flavour: contiguous chunks, no index
    cfg.context_parallel_algo = CP.ULYSSES
    out, idx = CP.get_batch_on_this_cp_rank(cfg, {"tokens": x}, cp_rank=1)
    assert idx is None and out["tokens"][0].tolist() == list(range(12, 24))
    # ring degree of the three algorithms
    assert CP.get_ring_degree(SimpleNamespace(context_parallel_size=1)) == 1
    assert CP.get_ring_degree(SimpleNamespace(context_parallel_size=4, context_parallel_algo=CP.RING)) == 4
    assert CP.get_ring_degree(SimpleNamespace(context_parallel_size=4, context_parallel_algo=CP.ULYSSES)) == 1
    hybrid = SimpleNamespace(context_parallel_size=4, context_parallel_algo="hybrid_cp_algo", ulysses_degree_in_cp=2)
    assert CP.get_ring_degree(hybrid) == 2
    hybrid.ulysses_degree_in_cp = 4
    with pytest.raises(ValueError):
        CP.get_ring_degree(hybrid)


def _cp_gather_worker(rank, world):
    full = torch.arange(48, dtype=torch.float32).reshape(2, 24)
    cu = torch.tensor([0, 8, 24], dtype=torch.int32)
    mine = full.index_select(1, CP.zigzag_index_packed(cu, world, rank))
    assert torch.equal(CP.gather_cp_outputs(mine, world, None, cu, ring=True), full)
    assert torch.equal(CP.get_tensor_allgather_cp_with_pack(mine, world, 1, None, cu), full)
    mine = full.index_select(1, CP.zigzag_index_plain(24, world, rank))
    assert torch.equal(CP.get_tensor_allgather_cp_without_pack(mine, world, 1), full)
    mine = full.chunk(world, dim=1)[rank].clone().requires_grad_(True)
    out = CP.gather_cp_outputs(mine, world)
    assert torch.equal(out.detach(), full)
    out.sum().backward()                                            # autograd flows through the local slice only
    assert torch.equal(mine.grad, torch.ones_like(mine))


def test_context_parallel_gather_restores_global_order():
    run_distributed(_cp_gather_worker, 2)


def _logprob_oracle(logits, labels):
    lsm = torch.log_softmax(logits.double(), -1)
    lp = lsm.gather(-1, labels.unsqueeze(-1)).squeeze(-1)
    ent = -(lsm.exp() * lsm).sum(-1)
    return lp, ent


def test_log_probs_and_entropy_single_rank_with_gradients():
    torch.manual_seed(0)
    logits = torch.randn(3, 7, 50, dtype=torch.float64, requires_grad=True)
    labels = torch.randint(0, 50, (3, 7))
    lp, ent = U.log_probs_and_entropy(logits, labels)
    want_lp, want_ent = _logprob_oracle(logits, labels)
    assert torch.allclose(lp.double(), want_lp, atol=1e-5) and torch.allclose(ent.double(), want_ent, atol=1e-5)
    w1, w2 = torch.randn(3, 7, dtype=torch.float64), torch.randn(3, 7, dtype=torch.float64)
    (g,) = torch.autograd.grad((lp * w1).sum() + (ent * w2).sum(), logits)
    (gw,) = torch.autograd.grad((want_lp * w1).sum() + (want_ent * w2).sum(), logits)
    assert torch.allclose(g, gw, atol=1e-5)
    assert U.log_probs_and_entropy(logits, labels, want_entropy=False)[1] is None
    assert torch.equal(U.compute_log_probs(logits, labels), U.vocab_parallel_log_probs(logits, labels))


def _vocab_parallel_worker(rank, world):
    torch.manual_seed(1)
    full = torch.randn(2, 5, 64, dtype=torch.float64)
    labels = torch.randint(0, 64, (2, 5))
    w1, w2 = torch.randn(2, 5, dtype=torch.float64), torch.randn(2, 5, dtype=torch.float64)
    ref = full.clone().requires_grad_(True)
    want_lp, want_ent = _logprob_oracle(ref, labels)
    (gw,) = torch.autograd.grad((want_lp * w1).sum() + (want_ent * w2).sum(), ref)
    part = 64 // world
    shard = full[..., rank * part:(rank + 1) * part].clone().requires_grad_(True)
    lp, ent = U.log_probs_and_entropy(shard, labels, dist.group.WORLD)
    assert torch.allclose(lp.double(), want_lp, atol=1e-5) and torch.allclose(ent.double(), want_ent, atol=1e-5)
    (g,) = torch.autograd.grad((lp * w1).sum() + (ent * w2).sum(), shard)
    assert torch.allclose(g, gw[..., rank * part:(rank + 1) * part], atol=1e-5)


def test_log_probs_and_entropy_over_a_sharded_vocabulary():
    run_distributed(_vocab_parallel_worker, 2)


def test_kl_penalties():
    lp, ref = torch.tensor([-1.0, -2.0, -30.0]), torch.tensor([-1.5, -1.0, -1.0])
    assert torch.allclose(U.compute_kl_penalty(lp, ref, "kl"), lp - ref)
    assert torch.allclose(U.compute_kl_penalty(lp, ref, "abs"), (lp - ref).abs())
    assert torch.allclose(U.compute_kl_penalty(lp, ref, "mse"), 0.5 * (lp - ref) ** 2)
    k3 = U.compute_kl_penalty(lp, ref, "low_var_kl")
    k = ref - lp
    assert torch.allclose(k3[:2], torch.exp(k[:2]) - k[:2] - 1)
    assert float(k3[2]) == 10.0                                   # exponent clamped at 20, value at 10
    with pytest.raises(NotImplementedError):
        U.compute_kl_penalty(lp, ref, "nope")


def test_samplers_cover_their_slices_and_resume():
    from mindspeed_rl_b200.datasets.dataloader import PretrainingSampler, PromptSampler
    assert list(PromptSampler(10, 0, 4)) == [[0, 1, 2, 3], [4, 5, 6, 7]]
    assert list(PromptSampler(10, 4, 4, drop_last=False)) == [[4, 5, 6, 7], [8, 9]]      # resume after 4 samples
    with pytest.raises(ValueError):
        PromptSampler(10, 10, 4)
    with pytest.raises(ValueError):
        PromptSampler(0, 0, 4)
    per_rank = [list(PretrainingSampler(12, 0, 2, r, 3)) for r in range(3)]
    assert per_rank[0] == [[0, 1], [6, 7]] and per_rank[1] == [[2, 3], [8, 9]] and per_rank[2] == [[4, 5], [10, 11]]
    assert list(PretrainingSampler(12, 6, 2, 1, 3)) == [[8, 9]]
    assert list(PretrainingSampler(8, 0, 2, 0, 3, drop_last=False)) == [[0, 1], [6, 7]]
    with pytest.raises(ValueError):
        PretrainingSampler(8, 0, 2, 3, 3)


def test_host_resident_optimizer_state_steps_in_chunks():
    """Optimizer state kept on the host and streamed through staging buffers chunk by chunk (the last chunk
    partial, two buffers of different size sharing the staging space) follows torch's AdamW; master weights can
    be refreshed from externally changed parameters; the state survives a checkpoint round trip."""
    from mindspeed_rl_b200.optim.distributed_optimizer import DistributedOptimizer
    from mindspeed_rl_b200.parallel.ddp import DistributedDataParallel
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(37, 53), torch.nn.Linear(53, 11))
    ref = torch.nn.Sequential(torch.nn.Linear(37, 53), torch.nn.Linear(53, 11))
    ref.load_state_dict(net.state_dict())
    ddp = DistributedDataParallel(net, None, 1)
    opt = DistributedOptimizer(ddp.buffers, lr=1e-2, betas=(0.9, 0.95), weight_decay=0.01, clip_grad=0.0,
                               offload_to_host=True, swap_chunks=5)
    ropt = torch.optim.AdamW(ref.parameters(), lr=1e-2, betas=(0.9, 0.95), weight_decay=0.01)

    def one_step(seed):
        x = torch.randn(6, 37, generator=torch.Generator().manual_seed(seed))
        ddp.zero_grad_buffer()
        net(x).pow(2).mean().backward()
        for p in net.parameters():
            p.main_grad.copy_(p.grad)
            p.grad = None
        ddp.finish_grad_sync(to_shards=True)
        opt.step()
        ropt.zero_grad()
        ref(x).pow(2).mean().backward()
        ropt.step()

    for step in range(3):
        one_step(step)
    for a, b in zip(net.parameters(), ref.parameters()):
        assert torch.allclose(a, b, atol=1e-6), (a - b).abs().max()
    n = sum(p.numel() for p in net.parameters())
    assert opt._stage[0]["master"].numel() < n                      # really chunked
    # parameters changed from outside (a checkpoint load): the master copy follows on request
    with torch.no_grad():
        for p, q in zip(net.parameters(), ref.parameters()):
            p.mul_(0.5)
            q.mul_(0.5)
    opt.reload_model_params()
    one_step(10)
    for a, b in zip(net.parameters(), ref.parameters()):
        assert torch.allclose(a, b, atol=1e-6)
    # state round trip into a fresh optimizer
    sd = opt.state_dict()
    opt2 = DistributedOptimizer(ddp.buffers, lr=1e-2, betas=(0.9, 0.95), weight_decay=0.01, clip_grad=0.0,
                                offload_to_host=True, swap_chunks=3)
    opt2.load_state_dict(sd)
    assert opt2.step_count == opt.step_count
    for a, b in zip(opt.state, opt2.state):
        for k in a:
            assert torch.equal(a[k], b[k]), k


def test_store_hands_out_token_balanced_batches():
    """With sequence-length balancing a consumer's draws are equal-sized parts of similar token count (rows, or
    whole groups of samples), and every row is handed out exactly once."""
    from mindspeed_rl_b200.data.transfer_dock import GRPOTransferDock, put_prompts_experience
    lens = [10, 200, 30, 180, 50, 160, 70, 140]
    td = GRPOTransferDock(8, 1)
    data, idx = put_prompts_experience({"prompts": [torch.arange(n) for n in lens]}, 1)
    td.put_experience(data, idx)
    td.put_experience({"responses": [torch.ones(3, dtype=torch.int64)] * 8,
                       "response_length": [torch.tensor([3], dtype=torch.int32)] * 8}, idx)
    sums, seen = [], []
    for _ in range(2):
        _, got = td.get_experience("actor_train", ["prompts", "prompt_length", "responses", "response_length"], 4,
                                   get_n_samples=False, use_batch_seqlen_balance=True)
        sums.append(sum(lens[i] for i in got))
        seen += got
    assert sorted(seen) == list(range(8)) and abs(sums[0] - sums[1]) <= 40, sums       # total 840: about 420 each
    assert td.all_consumed("actor_train")
    # groups of two samples stay together
    td = GRPOTransferDock(4, 2)
    data, idx = put_prompts_experience({"prompts": [torch.arange(n) for n in (10, 200, 190, 20)]}, 2)
    td.put_experience(data, idx)
    td.put_experience({"responses": [torch.ones(2, dtype=torch.int64)] * 8,
                       "response_length": [torch.tensor([2], dtype=torch.int32)] * 8}, idx)
    _, got = td.get_experience("actor_train", ["prompts", "prompt_length", "responses", "response_length"], 4,
                               get_n_samples=True, use_batch_seqlen_balance=True)
    groups = sorted({i // 2 for i in got})
    assert len(got) == 4 and got == [g * 2 + j for g in groups for j in range(2)]
    assert sorted(groups) in ([0, 1], [2, 3], [0, 2], [1, 3])        # one short and one long prompt group


def test_small_helpers_partition_filter_builder_and_tool_file(tmp_path):
    import numpy as np
    from mindspeed_rl_b200.datasets.indexed_dataset import (IndexedDataset, IndexedDatasetBuilder, get_bin_path,
                                                            get_idx_path)
    from mindspeed_rl_b200.tools.base import load_tool_map
    from mindspeed_rl_b200.utils.seqlen_balancing import heapq_partition

    parts = heapq_partition([9, 1, 8, 2, 7, 3], 2, equal_size=True)
    assert sorted(map(len, parts)) == [3, 3] and sorted(i for p in parts for i in p) == list(range(6))
    sums = [sum([9, 1, 8, 2, 7, 3][i] for i in p) for p in parts]
    assert abs(sums[0] - sums[1]) <= 2
    assert sorted(map(len, heapq_partition([5, 5, 5], 2, equal_size=False))) == [1, 2]
    with pytest.raises(ValueError):
        heapq_partition([1, 2, 3], 2, equal_size=True)

    prefix = str(tmp_path / "docs")
    b = IndexedDatasetBuilder(get_bin_path(prefix), dtype=np.int32)
    b.add_document(torch.arange(7), [3, 4])                 # one document of two sequences
    b.add_item(np.arange(10))
    b.end_document()
    b.finalize(get_idx_path(prefix))
    ds = IndexedDataset(prefix)
    assert len(ds) == 3 and ds[0].tolist() == [0, 1, 2] and ds[1].tolist() == [3, 4, 5, 6]
    assert ds.document_indices.tolist() == [0, 2, 3] and ds.get_filter_mask().all()
    short = IndexedDataset(prefix, max_len=4) if "max_len" in IndexedDataset.__init__.__code__.co_varnames else None
    if short is not None:
        mask = short.get_filter_mask()
        assert mask.tolist() == [True, True, False]
        short.do_filter(mask)
        assert len(short) == 2 and short.sequence_lengths.tolist() == [3, 4]

    tools = load_tool_map(os.path.join(os.path.dirname(__file__), "..", "configs", "tools", "retool.yaml"))
    assert list(tools) == ["code_interpreter"] and type(tools["code_interpreter"]).__name__ == "ReTool"
    assert tools["code_interpreter"].schema.to_openai()["function"]["parameters"]["required"] == ["code"]


def test_expert_bias_follows_the_load():
    """Auxiliary-loss-free balancing: experts that received fewer tokens than the mean since the last update get a
    higher routing bias, the others a lower one, and the counters restart."""
    from mindspeed_rl_b200.models.gpt import GPTModel, PackedMeta
    from mindspeed_rl_b200.models.transformer_config import TransformerConfig
    cfg = TransformerConfig(num_layers=1, hidden_size=32, ffn_hidden_size=64, num_attention_heads=4, num_query_groups=2,
                            vocab_size=64, params_dtype=torch.float32, num_experts=4, moe_router_topk=2,
                            moe_ffn_hidden_size=16, moe_router_enable_expert_bias=True, max_position_embeddings=64)
    model = GPTModel(cfg, device="cpu", seed=1)
    moe = model.decoder.layers[0].mlp
    ids = torch.randint(0, 64, (24,), generator=torch.Generator().manual_seed(0))
    lp, _ = model.forward_logprob(ids, ids, PackedMeta.from_lengths([24], "cpu"))
    lp.sum().backward()
    load = moe._load_since_update.clone()
    assert float(load.sum()) == 24 * 2 and moe.router.expert_bias.abs().sum() == 0
    moe.update_expert_bias(rate=0.01)
    want = 0.01 * torch.sign(load.mean() - load)
    assert torch.allclose(moe.router.expert_bias, want) and float(moe._load_since_update.sum()) == 0
    with torch.no_grad():                                     # forward-only passes do not count as training load
        model.forward_logprob(ids, ids, PackedMeta.from_lengths([24], "cpu"))
    assert float(moe._load_since_update.sum()) == 0


def test_metric_sinks_with_stand_in_packages(monkeypatch, tmp_path):
    """The Weights & Biases and SwanLab sinks forward numeric metrics with the step; a missing package only
    disables the sink."""
    import sys
    import types
    from mindspeed_rl_b200.obs import loggers

    calls = {}

    def fake(name):
        mod = types.ModuleType(name)
        mod.init = lambda **kw: calls.setdefault(name + ".init", kw) or object()
        mod.log = lambda data, step=None: calls.setdefault(name + ".log", []).append((data, step))
        return mod

    monkeypatch.setitem(sys.modules, "wandb", fake("wandb"))
    monkeypatch.setitem(sys.modules, "swanlab", fake("swanlab"))
    w = loggers.WandbLogger({"wandb_project": "p", "wandb_exp_name": "e", "wandb_save_dir": str(tmp_path / "w")})
    s = loggers.SwanLabLogger({"swanlab_project": "p", "swanlab_exp_name": "e", "swanlab_save_dir": str(tmp_path / "s")})
    for sink in (w, s):
        sink.log_metrics({"a": 1.5, "b": 2, "text": "skip me"}, 7)
    assert calls["wandb.init"]["project"] == "p" and calls["wandb.init"]["name"].startswith("e-")
    assert calls["wandb.log"] == [({"a": 1.5, "b": 2}, 7)] and calls["swanlab.log"] == [({"a": 1.5, "b": 2}, 7)]
    assert calls["swanlab.init"]["experiment_name"] == "e" and calls["swanlab.init"]["mode"] == "local"
    monkeypatch.setitem(sys.modules, "wandb", None)            # import fails: the sink switches itself off
    off = loggers.WandbLogger({})
    off.log_metrics({"a": 1.0}, 1)
    assert off.run is None


def test_static_row_ranges_for_ordered_consumption():
    from mindspeed_rl_b200.trainer.compute_utils import get_current_dp_range_indexes
    assert get_current_dp_range_indexes(2, 6) == [[0, 1], [2, 3], [4, 5]]
    assert get_current_dp_range_indexes(3, 6, current_dp_rank=1) == [[6, 7, 8], [9, 10, 11]]


def test_store_waits_for_late_cells_and_gives_up_on_missing_ones(capsys):
    """A read of explicitly named rows waits for cells that a slow producer fills later, reports that it is
    waiting once the first limit has passed, and raises after ten times the limit when a cell never arrives."""
    import threading
    import time
    from mindspeed_rl_b200.data.transfer_dock import GRPOTransferDock, put_prompts_experience
    td = GRPOTransferDock(2, 1, timeout=0.05, timeout_interval=0.05)
    data, idx = put_prompts_experience({"prompts": [torch.arange(3), torch.arange(5)]}, 1)
    td.put_experience(data, idx)

    def late():
        time.sleep(0.2)
        td.put_experience({"responses": [torch.tensor([7]), torch.tensor([8, 9])]}, [0, 1])

    t = threading.Thread(target=late)
    t.start()
    batch, got = td.get_experience("actor_train", ["responses"], 2, indexes=[0, 1], get_n_samples=False)
    t.join()
    assert got == [0, 1] and batch["responses"].tolist() == [[7, 0], [8, 9]]
    assert "waiting" in capsys.readouterr().out                     # the wait was reported while it lasted
    t0 = time.time()
    with pytest.raises(TimeoutError):
        td.get_experience("actor_train", ["old_log_prob"], 2, indexes=[0, 1], get_n_samples=False)
    assert 0.4 < time.time() - t0 < 5.0
    with pytest.raises(ValueError):
        td.get_experience("actor_train", ["responses"], 2, indexes=[0, 5], get_n_samples=False)
    with pytest.raises(ValueError):
        td.put_experience({"responses": [torch.tensor([1])]}, [0, 1])          # one row for two indexes
    with pytest.raises(ValueError):
        td.put_experience({"responses": [torch.tensor([1])]}, [9])


def test_yarn_frequencies_match_the_transformers_formula():
    """Rotary frequencies under YaRN scaling (DeepSeek-style long context) against the implementation in
    the transformers package, and the scaled table's amplitude."""
    from mindspeed_rl_b200.ops.elementwise import _yarn_inv_freq, rope_table
    hd, theta = 64, 10000.0
    sc = dict(factor=40.0, original_max_position_embeddings=4096, beta_fast=32, beta_slow=1, mscale=1.0,
              mscale_all_dim=1.0)
    inv = 1.0 / (theta ** (torch.arange(0, hd // 2, dtype=torch.float64) * 2.0 / hd))
    new, mscale = _yarn_inv_freq(inv, hd, theta, sc)
    assert mscale == 1.0                                              # equal mscale factors cancel
    assert torch.allclose(new[:4], inv[:4]) and torch.allclose(new[-4:], inv[-4:] / 40.0)   # fast dims kept, slow ones stretched
    assert bool((new[1:] <= new[:-1]).all())
    _, only_m = _yarn_inv_freq(inv, hd, theta, dict(sc, mscale_all_dim=0.0))
    assert only_m == pytest.approx(0.1 * math.log(40.0) + 1.0)
    try:
        from transformers import PretrainedConfig
        from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS
        cfg = PretrainedConfig()
        cfg.rope_theta, cfg.hidden_size, cfg.num_attention_heads, cfg.head_dim = theta, hd * 4, 4, hd
        cfg.max_position_embeddings = 4096 * 40
        cfg.rope_scaling = dict(sc, rope_type="yarn")
        cfg.rope_parameters = dict(cfg.rope_scaling, rope_theta=theta)
        inv_hf, att = ROPE_INIT_FUNCTIONS["yarn"](cfg, "cpu")
    except Exception as e:                                            # another transformers API: nothing to compare with
        pytest.skip(f"transformers rope helpers not usable here: {e!r}")
    assert float((inv_hf.double() - new).abs().max()) < 1e-7 and att == pytest.approx(mscale)
    tab = rope_table(32, hd, theta, "cpu", dict(sc, mscale_all_dim=0.0))
    assert tab.shape == (32, hd) and float(tab[0, 0]) == pytest.approx(only_m, rel=1e-6)   # cos(0) x amplitude


def test_decode_groups_for_the_shared_prefix_path():
    from mindspeed_rl_b200.ops.decode import build_decode_groups, decode_group_max
    # rows 0-2 and 4 sample prompt "a" (prefix 37 keys), row 3 is alone, rows 5-6 sample prompt "b"
    ids = ["a", "a", "a", "c", "a", "b", "b"]
    plen = [37, 37, 37, 50, 37, 20, 21]
    key_start, rows, prefix, shared = build_decode_groups(ids, plen, group_max=3, multiple=16)
    assert shared and len(rows) == len(prefix) == 7 and all(len(r) == 8 for r in rows)
    assert rows[0][:3] == [0, 1, 2] and rows[0][3:] == [-1] * 5 and prefix[0] == 32       # 37 rounded down to the tile
    assert rows[1][:1] == [4] and prefix[1] == 0                                         # overflow of the group: alone
    assert rows[2][:1] == [3] and prefix[2] == 0
    assert rows[3][:2] == [5, 6] and prefix[3] == 16                                     # min(20, 21) rounded down
    assert rows[4:] == [[-1] * 8] * 3 and prefix[4:] == [0, 0, 0]
    assert key_start == [32, 32, 32, 0, 0, 16, 16]
    _, _, p1, s1 = build_decode_groups(ids, [5] * 7, group_max=8, multiple=16)
    assert not s1 and set(p1) == {0}                                                     # prefixes shorter than a tile
    assert decode_group_max(28, 4) == 8 and decode_group_max(32, 2) == 4 and decode_group_max(64, 1, 64) == 2
