"""Multi-rank behaviour on CPU (gloo): parallel-state rank maths, tensor/sequence-parallel model
equivalence with the single-rank model, distributed optimizer vs single-rank Adam, expert
parallel MoE, and the experience store served over RPC."""
import os

import torch
import torch.distributed as dist

from dist_utils import run_distributed
from mindspeed_rl_b200.parallel.state import RankLayout


def test_rank_layout_groups():
    lay = RankLayout(16, tp=2, pp=2, cp=2)
    assert lay.dp == 2
    assert lay.groups("tp")[0] == [0, 1] and lay.groups("cp")[0] == [0, 2]
    assert lay.groups("dp")[0] == [0, 4] and lay.groups("pp")[0] == [0, 8]
    assert lay.coords(13) == {"tp": 1, "cp": 0, "dp": 1, "pp": 1}
    assert lay.rank_of(tp=1, cp=0, dp=1, pp=1) == 13
    moe = RankLayout(8, tp=2, ep=2, moe_tp_extend_ep=True)
    assert moe.ep_total == 4 and moe.expert_tp == 1 and moe.expert_dp == 2
    assert moe.expert_groups("ep")[0] == [0, 1, 2, 3]


def _shard_state(full, cfg, tp, r):
    from mindspeed_rl_b200.checkpoint import convert as C
    nkv = cfg.num_query_groups
    out = {}
    for k, v in full.items():
        if k.endswith("linear_qkv.weight") or k.endswith("linear_qkv.bias"):
            out[k] = C.shard_qkv(v, nkv, tp, r)
        elif k.endswith("linear_fc1.weight"):
            g, u = v.chunk(2, 0)
            out[k] = C.shard_fc1(g, u, tp, r)
        elif k.endswith(("linear_q_up_proj.weight", "linear_kv_up_proj.weight", "linear_q_proj.weight")):
            out[k] = C.shard_rows(v, tp, r)          # latent attention: head-major rows
        elif k.endswith("linear_proj.weight") or k.endswith("linear_fc2.weight"):
            out[k] = C.shard_cols(v, tp, r)
        elif k.endswith("word_embeddings.weight") or k.endswith("output_layer.weight"):
            out[k] = C.shard_rows(v, tp, r)
        else:
            out[k] = v.clone()
    return out


def _tp_worker(rank, world, sp):
    from mindspeed_rl_b200.models.gpt import GPTModel, PackedMeta
    from mindspeed_rl_b200.models.transformer_config import TransformerConfig
    from mindspeed_rl_b200.parallel.state import initialize_model_parallel
    from mindspeed_rl_b200.parallel.tp_comm import TPComm
    ps = initialize_model_parallel(tensor_model_parallel_size=world)
    kw = dict(num_layers=2, hidden_size=32, ffn_hidden_size=64, num_attention_heads=4, num_query_groups=2,
              vocab_size=64, add_qkv_bias=True, params_dtype=torch.float32, max_position_embeddings=128)
    torch.manual_seed(0)
    full = GPTModel(TransformerConfig(**kw), device="cpu", seed=5)
    cfg = TransformerConfig(tensor_model_parallel_size=world, sequence_parallel=sp, **kw)
    comm = TPComm(ps.group("tp"), sp, world_size=world, rank=rank)
    model = GPTModel(cfg, comm, device="cpu")
    model.load_state_dict(_shard_state(full.state_dict(), cfg, world, rank))
    lens = [6, 10]
    meta = PackedMeta.from_lengths(lens, "cpu", align=world)
    t = int(meta.cu_seqlens[-1])
    g = torch.Generator().manual_seed(1)
    ids, labels, w = torch.randint(0, 64, (t,), generator=g), torch.randint(0, 64, (t,), generator=g), torch.randn(t, generator=g)
    ref_lp, ref_ent = full.forward_logprob(ids, labels, meta, 0.9, True)
    (ref_lp * w + 0.1 * ref_ent).sum().backward()
    if sp:   # activations between layers are sharded over tokens
        model.embed = lambda x, _m=model: _seq_shard(_orig_embed(_m, x), world, rank)
    lp, ent = model.forward_logprob(ids, labels, meta, 0.9, True)
    (lp * w + 0.1 * ent).sum().backward()
    assert torch.allclose(lp, ref_lp, atol=1e-4), (lp - ref_lp).abs().max()
    assert torch.allclose(ent, ref_ent, atol=1e-4)
    want = _shard_state({n: p.grad for n, p in full.named_parameters()}, cfg, world, rank)
    for n, p in model.named_parameters():
        g_ = p.grad
        if sp and p.dim() == 1 and "linear_qkv" not in n:   # norm weights see only the local tokens
            dist.all_reduce(g_)
        assert torch.allclose(g_, want[n], atol=2e-4, rtol=1e-3), (n, (g_ - want[n]).abs().max())


def _orig_embed(m, ids):
    from mindspeed_rl_b200.models.gpt import _EmbedFn
    from mindspeed_rl_b200.parallel.tp_comm import TPComm
    plain = TPComm(m.comm.group, False, world_size=m.comm.world_size, rank=m.comm.rank)
    return _EmbedFn.apply(m.embedding.word_embeddings.weight, ids, plain, m.vocab_start)


class _Shard(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, world, rank):
        ctx.world, ctx.rank = world, rank
        return x.chunk(world, 0)[rank].contiguous()

    @staticmethod
    def backward(ctx, d):
        parts = [torch.zeros_like(d) for _ in range(ctx.world)]
        dist.all_gather(parts, d.contiguous())
        return torch.cat(parts, 0), None, None


def _seq_shard(x, world, rank):
    return _Shard.apply(x, world, rank)


def test_tensor_parallel_matches_single_rank():
    run_distributed(_tp_worker, 2, False)


def test_sequence_parallel_matches_single_rank():
    run_distributed(_tp_worker, 2, True)


def _zero1_worker(rank, world, pipelined_gather=False):
    from mindspeed_rl_b200.optim.distributed_optimizer import DistributedOptimizer
    from mindspeed_rl_b200.parallel.ddp import DistributedDataParallel
    from mindspeed_rl_b200.parallel.state import initialize_model_parallel
    ps = initialize_model_parallel()
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(16, 24), torch.nn.Linear(24, 8))
    ref = torch.nn.Sequential(torch.nn.Linear(16, 24), torch.nn.Linear(24, 8))
    ref.load_state_dict(net.state_dict())
    ddp = DistributedDataParallel(net, ps.group("dp_cp"), world)
    opt = DistributedOptimizer(ddp.buffers, lr=1e-2, betas=(0.9, 0.95), weight_decay=0.01, clip_grad=0.5,
                               dp_group=ps.group("dp_cp"), dp_rank=rank, overlap_param_gather=pipelined_gather,
                               gather_chunks=3)
    ropt = torch.optim.AdamW(ref.parameters(), lr=1e-2, betas=(0.9, 0.95), weight_decay=0.01)
    for step in range(3):
        xs = [torch.randn(4, 16, generator=torch.Generator().manual_seed(10 * step + r)) for r in range(world)]
        ddp.zero_grad_buffer()
        out = net(xs[rank]).pow(2).mean()
        out.backward()
        for p in net.parameters():          # plain autograd grads -> flat buffer
            p.main_grad.copy_(p.grad)
            p.grad = None
        ddp.finish_grad_sync(to_shards=True)
        opt.step()
        ropt.zero_grad()
        (sum(ref(x).pow(2).mean() for x in xs) / world).backward()
        torch.nn.utils.clip_grad_norm_(ref.parameters(), 0.5)
        ropt.step()
    for a, b in zip(net.parameters(), ref.parameters()):
        assert torch.allclose(a, b, atol=1e-5), (a - b).abs().max()


def _overlap_worker(rank, world):
    """Bucketed gradient reduction started from the layers' backward (last micro-batch only) gives the
    parameters of the plain reduce-after-backward path, bucket by bucket in backward order."""
    from mindspeed_rl_b200.models.gpt import GPTModel, PackedMeta
    from mindspeed_rl_b200.models.training_engine import TrainingEngine
    from mindspeed_rl_b200.models.transformer_config import TransformerConfig
    from mindspeed_rl_b200.optim.distributed_optimizer import DistributedOptimizer
    from mindspeed_rl_b200.parallel.ddp import DistributedDataParallel
    from mindspeed_rl_b200.parallel.state import initialize_model_parallel
    ps = initialize_model_parallel()
    cfg = TransformerConfig(num_layers=3, hidden_size=32, ffn_hidden_size=64, num_attention_heads=4, num_query_groups=2,
                            vocab_size=64, params_dtype=torch.float32, max_position_embeddings=64)
    results = []
    for overlap in (False, True):
        core = GPTModel(cfg, device="cpu", seed=11)
        ddp = DistributedDataParallel(core, ps.group("dp_cp"), world)
        launched = []
        if overlap:
            ddp.enable_grad_overlap(bucket_numel=4000)
            assert len(ddp.buffers[0].bucket_ranges) >= 3
            orig = ddp._launch_bucket
            ddp._launch_bucket = lambda bi, k: (launched.append((bi, k)), orig(bi, k))[1]
        opt = DistributedOptimizer(ddp.buffers, lr=1e-2, betas=(0.9, 0.95), weight_decay=0.0, clip_grad=1.0,
                                   dp_group=ps.group("dp_cp"), dp_rank=rank)
        g = torch.Generator().manual_seed(5 + rank)
        for step in range(2):
            ddp.zero_grad_buffer()
            for micro in range(2):                      # gradients accumulate; only the last micro-batch overlaps
                meta = PackedMeta.from_lengths([7, 5], "cpu")
                ids, labels = torch.randint(0, 64, (12,), generator=g), torch.randint(0, 64, (12,), generator=g)
                if micro == 1:
                    ddp.begin_last_microbatch()
                lp, _ = core.forward_logprob(ids, labels, meta, 1.0, False)
                (-lp.mean()).backward()
            ddp.finish_grad_sync(to_shards=True)
            opt.step()
        if overlap:
            # 3 layer buckets (or more) per step went out during the backward, last layers first
            assert len(launched) >= 2 * 2 and launched[0][1] <= launched[1][1]
        results.append(torch.cat([p.detach().reshape(-1) for p in core.parameters()]))
    assert torch.allclose(results[0], results[1], atol=1e-6), (results[0] - results[1]).abs().max()


def test_overlapped_bucketed_grad_reduce_matches_plain():
    run_distributed(_overlap_worker, 2)


def test_distributed_optimizer_matches_adamw():
    run_distributed(_zero1_worker, 2)
    run_distributed(_zero1_worker, 2, True)        # shard updated in chunks, chunks gathered behind the update


def _ep_worker(rank, world):
    from mindspeed_rl_b200.models.gpt import GPTModel, PackedMeta
    from mindspeed_rl_b200.models.transformer_config import TransformerConfig
    from mindspeed_rl_b200.parallel.state import initialize_model_parallel, set_parallel_state
    kw = dict(num_layers=1, hidden_size=32, ffn_hidden_size=64, num_attention_heads=4, num_query_groups=2,
              vocab_size=64, params_dtype=torch.float32, max_position_embeddings=64, num_experts=4,
              moe_router_topk=2, moe_ffn_hidden_size=16, norm_topk_prob=True, moe_aux_loss_coeff=0.0)
    set_parallel_state(None)
    full = GPTModel(TransformerConfig(**kw), device="cpu", seed=3)       # all experts on one rank
    initialize_model_parallel(expert_model_parallel_size=world)
    model = GPTModel(TransformerConfig(expert_model_parallel_size=world, **kw), device="cpu", seed=3)
    sd = full.state_dict()
    per = 4 // world
    for k in list(sd):
        if k.endswith("experts.weight1"):
            sd[k] = sd[k].view(32, 4, 32)[:, rank * per:(rank + 1) * per].reshape(32, -1).contiguous()
        if k.endswith("experts.weight2"):
            sd[k] = sd[k].view(4, 16, 32)[rank * per:(rank + 1) * per].reshape(-1, 32).contiguous()
    model.load_state_dict(sd)
    # every rank feeds different tokens (data parallel over the EP group)
    g = torch.Generator().manual_seed(100 + rank)
    meta = PackedMeta.from_lengths([9], "cpu")
    ids, labels = torch.randint(0, 64, (9,), generator=g), torch.randint(0, 64, (9,), generator=g)
    ref, _ = full.forward_logprob(ids, labels, meta)
    ref.sum().backward()
    lp, _ = model.forward_logprob(ids, labels, meta)
    lp.sum().backward()
    assert torch.allclose(lp, ref, atol=1e-4), (lp - ref).abs().max()
    # expert grads: sum over the ranks' tokens equals the sum of single-rank grads over both inputs
    gw = model.decoder.layers[0].mlp.experts.weight2.grad
    fw = full.decoder.layers[0].mlp.experts.weight2.grad.view(4, 16, 32).clone()
    dist.all_reduce(fw)
    assert torch.allclose(gw.view(per, 16, 32), fw[rank * per:(rank + 1) * per], atol=2e-4)
    # a peer-memory dispatcher that reports a slab overflow (dispatch -> None on every member) sends the
    # layer to the all-to-all path: same result
    class _Overflowing:
        calls = 0

        def dispatch(self, x, idx):
            _Overflowing.calls += 1
            return None

    moe = model.decoder.layers[0].mlp
    moe._p2p_dispatcher = lambda x: _Overflowing()
    with torch.no_grad():
        lp2, _ = model.forward_logprob(ids, labels, meta)
    assert _Overflowing.calls == 1 and torch.allclose(lp2, lp.detach(), atol=1e-6)


def test_expert_parallel_matches_single_rank():
    run_distributed(_ep_worker, 2)


def _ep_optimizer_worker(rank, world, tmp):
    """One optimizer step with EP=2 (experts differ per rank, dense weights are replicated) equals the
    step of a single-rank model that holds all experts and sees both ranks' tokens; a checkpoint
    written afterwards reloads into a fresh model with every rank's own experts."""
    from mindspeed_rl_b200.checkpoint.mcore import load_checkpoint, save_checkpoint
    from mindspeed_rl_b200.models.gpt import GPTModel, PackedMeta
    from mindspeed_rl_b200.models.transformer_config import TransformerConfig
    from mindspeed_rl_b200.optim.distributed_optimizer import DistributedOptimizer
    from mindspeed_rl_b200.parallel.ddp import DistributedDataParallel, expert_replica_groups
    from mindspeed_rl_b200.parallel.state import initialize_model_parallel, set_parallel_state
    kw = dict(num_layers=1, hidden_size=32, ffn_hidden_size=64, num_attention_heads=4, num_query_groups=2,
              vocab_size=64, params_dtype=torch.float32, max_position_embeddings=64, num_experts=4,
              moe_router_topk=2, moe_ffn_hidden_size=16, norm_topk_prob=True, moe_aux_loss_coeff=0.0)
    set_parallel_state(None)
    full = DistributedDataParallel(GPTModel(TransformerConfig(**kw), device="cpu", seed=3))
    full_opt = DistributedOptimizer(full.buffers, lr=1e-2, clip_grad=1e9, weight_decay=0.0)
    ps = initialize_model_parallel(expert_model_parallel_size=world)
    cfg = TransformerConfig(expert_model_parallel_size=world, **kw)

    def shard(sd):
        per, out = 4 // world, dict(sd)
        for k in list(out):
            if k.endswith("experts.weight1"):
                out[k] = out[k].view(32, 4, 32)[:, rank * per:(rank + 1) * per].reshape(32, -1).contiguous()
            if k.endswith("experts.weight2"):
                out[k] = out[k].view(4, 16, 32)[rank * per:(rank + 1) * per].reshape(-1, 32).contiguous()
        return out

    core = GPTModel(cfg, device="cpu", seed=3)
    core.load_state_dict(shard({k: v.clone() for k, v in full.module.state_dict().items()}))
    model = DistributedDataParallel(core, ps.group("dp_cp"), world, **expert_replica_groups(ps, cfg))
    assert any(b.is_expert for b in model.buffers) and len(model.buffers) == 2
    opt = DistributedOptimizer(model.buffers, lr=1e-2, clip_grad=1e9, weight_decay=0.0, dp_group=ps.group("dp_cp"),
                               dp_rank=ps.rank_in("dp_cp"), model_parallel_group=ps.group("mp"))
    meta = PackedMeta.from_lengths([9], "cpu")
    for r in range(world):                      # the single-rank model sees every rank's tokens
        g = torch.Generator().manual_seed(100 + r)
        ids, labels = torch.randint(0, 64, (9,), generator=g), torch.randint(0, 64, (9,), generator=g)
        (full.module.forward_logprob(ids, labels, meta)[0].sum() / world).backward()
        if r == rank:
            core.forward_logprob(ids, labels, meta)[0].sum().backward()
    for p in list(full.module.parameters()) + list(core.parameters()):
        if p.grad is not None:                  # layers accumulate into main_grad themselves
            p.main_grad.add_(p.grad)
    model.finish_grad_sync(to_shards=True)
    _, norm, _ = opt.step()
    _, full_norm, _ = full_opt.step()
    assert torch.allclose(norm, full_norm, rtol=1e-4), (norm, full_norm)
    want = shard(full.module.state_dict())
    for k, v in core.state_dict().items():
        assert torch.allclose(v, want[k], atol=2e-5), (k, (v - want[k]).abs().max())
    mine = core.decoder.layers[0].mlp.experts.weight2.detach().clone()
    both = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(both, mine)
    assert not torch.allclose(both[0], both[1]), "the expert-parallel ranks ended up with identical experts"
    # checkpoint round trip: every EP rank has a directory of its own
    save_checkpoint(tmp, 1, core, opt, None, ps, None)
    fresh = GPTModel(cfg, device="cpu", seed=77)
    load_checkpoint(tmp, fresh, None, None, ps, None)
    for k, v in fresh.state_dict().items():
        assert torch.equal(v, core.state_dict()[k]), k


def test_expert_parallel_optimizer_step_and_checkpoint(tmp_path):
    run_distributed(_ep_optimizer_worker, 2, str(tmp_path))


def _ep_rollout_worker(rank, world):
    """Expert-parallel rollout engines step together: a rank with fewer (or no) requests keeps
    joining the token exchanges, and every rank's greedy tokens equal the single-rank model's."""
    from mindspeed_rl_b200.models.gpt import GPTModel
    from mindspeed_rl_b200.models.transformer_config import TransformerConfig
    from mindspeed_rl_b200.parallel.state import initialize_model_parallel, set_parallel_state
    from mindspeed_rl_b200.reshard.alias import alias_rollout_weights
    from mindspeed_rl_b200.rollout.engine import LLMEngine
    from mindspeed_rl_b200.rollout.scheduler import SamplingParams
    kw = dict(num_layers=2, hidden_size=32, ffn_hidden_size=64, num_attention_heads=4, num_query_groups=2,
              vocab_size=64, params_dtype=torch.float32, max_position_embeddings=64, num_experts=4,
              moe_router_topk=2, moe_ffn_hidden_size=16, norm_topk_prob=True, moe_aux_loss_coeff=0.0)
    set_parallel_state(None)
    full = GPTModel(TransformerConfig(**kw), device="cpu", seed=3)
    for p in full.parameters():
        p.data.mul_(3.0)
    ps = initialize_model_parallel(expert_model_parallel_size=world)
    model = GPTModel(TransformerConfig(expert_model_parallel_size=world, **kw), device="cpu", seed=3)
    sd = full.state_dict()
    per = 4 // world
    for k in list(sd):
        if k.endswith("experts.weight1"):
            sd[k] = sd[k].view(32, 4, 32)[:, rank * per:(rank + 1) * per].reshape(32, -1).contiguous()
        if k.endswith("experts.weight2"):
            sd[k] = sd[k].view(4, 16, 32)[rank * per:(rank + 1) * per].reshape(-1, 32).contiguous()
    model.load_state_dict(sd)

    def engine(m, group):
        e = LLMEngine(m.cfg, "cpu", max_num_seqs=4, max_num_batched_tokens=64, max_model_len=32, block_size=4,
                      lockstep_group=group)
        e.runner.bind_weights(alias_rollout_weights(m))
        e.init_cache(32)
        return e
    prompts = [[3, 9, 27, 5], [1, 2, 3, 4, 5, 6], [11, 12]] if rank == 0 else []      # rank 1 has nothing to do
    params = SamplingParams(n=1, temperature=0.0, max_tokens=6)
    ep = engine(model, ps.group("ep"))
    got = [o.outputs[0].token_ids for o in ep.generate(prompts, params)]
    set_parallel_state(None)
    ref = [o.outputs[0].token_ids for o in engine(full, None).generate(prompts, params)]
    assert got == ref, (got, ref)
    if rank == 1:
        assert ep.stats.get("idle_steps", 0) > 0


def test_expert_parallel_rollout_steps_together():
    run_distributed(_ep_rollout_worker, 2)


def _ep_rehome_worker(rank, world):
    """Training EP2 (x expert-DP2) on four ranks; the rollout re-homes the experts to EP4, to one full copy per
    rank (EP1), and to an EP2 placement with a redundant expert slot per rank: greedy tokens always equal the
    single-rank model's."""
    from mindspeed_rl_b200.models.gpt import GPTModel
    from mindspeed_rl_b200.models.transformer_config import TransformerConfig
    from mindspeed_rl_b200.parallel.ddp import DistributedDataParallel, expert_replica_groups
    from mindspeed_rl_b200.parallel.state import initialize_model_parallel, set_parallel_state
    from mindspeed_rl_b200.reshard.alias import alias_rollout_weights
    from mindspeed_rl_b200.reshard.planner import Resharder
    from mindspeed_rl_b200.rollout.engine import LLMEngine
    from mindspeed_rl_b200.rollout.eplb import expert_map_from_counts
    from mindspeed_rl_b200.rollout.scheduler import SamplingParams
    kw = dict(num_layers=2, hidden_size=32, ffn_hidden_size=64, num_attention_heads=4, num_query_groups=2,
              vocab_size=64, params_dtype=torch.float32, max_position_embeddings=64, num_experts=4,
              moe_router_topk=2, moe_ffn_hidden_size=16, norm_topk_prob=True, moe_aux_loss_coeff=0.0)
    set_parallel_state(None)
    full = GPTModel(TransformerConfig(**kw), device="cpu", seed=3)
    for p in full.parameters():
        p.data.mul_(3.0)
    ps = initialize_model_parallel(expert_model_parallel_size=2)
    cfg = TransformerConfig(expert_model_parallel_size=2, **kw)
    model = GPTModel(cfg, device="cpu", seed=3)
    er = ps.rank_in("ep")
    sd = full.state_dict()
    for k in list(sd):
        if k.endswith("experts.weight1"):
            sd[k] = sd[k].view(32, 4, 32)[:, er * 2:(er + 1) * 2].reshape(32, -1).contiguous()
        if k.endswith("experts.weight2"):
            sd[k] = sd[k].view(4, 16, 32)[er * 2:(er + 1) * 2].reshape(-1, 32).contiguous()
    model.load_state_dict(sd)
    ddp = DistributedDataParallel(model, ps.group("dp_cp"), ps.size("dp_cp"), **expert_replica_groups(ps, cfg))
    assert len(ddp.buffers) == 2                             # dense + experts

    ref_engine = LLMEngine(full.cfg, "cpu", max_num_seqs=4, max_num_batched_tokens=64, max_model_len=32, block_size=4)
    ref_engine.runner.bind_weights(alias_rollout_weights(full))
    ref_engine.init_cache(32)
    prompts = [[3 + rank, 9, 27, 5], [1, 2, 3, 4, 5, 6 + rank]] if rank != 2 else []      # one rank has nothing to do
    params = SamplingParams(n=1, temperature=0.0, max_tokens=6)
    want = [o.outputs[0].token_ids for o in ref_engine.generate(prompts, params)] if prompts else []
    torch.manual_seed(1)
    emap = expert_map_from_counts(torch.randint(1, 50, (2, 4)), 2, 1)          # 2 ranks x (2 + 1) slots
    for infer_ep, mapping in ((4, None), (1, None), (2, emap)):
        r = Resharder(cfg, ddp, ps, 1, "cpu",
                      lambda icfg, comm: LLMEngine(icfg, "cpu", max_num_seqs=4, max_num_batched_tokens=64,
                                                   max_model_len=32, block_size=4),
                      infer_ep=infer_ep, expert_map=mapping)
        assert r.rehome and r.infer_state.size("ep") == infer_ep
        # the engines of a rollout expert-parallel group step together
        r.engine.lockstep_group, r.engine.lookahead_decode = r._lockstep_group(), False
        w = r.reshard(model)
        n_slots = (4 + (2 if mapping else 0)) // infer_ep
        assert w.layers[0].moe.num_local == n_slots and w.layers[0].moe.ep_size == infer_ep
        if mapping:
            assert w.layers[0].moe.log2phy.shape[0] == 4 and int((w.layers[0].moe.log2phy >= 0).sum()) == 6
        r.engine.runner.bind_weights(w)
        r.engine.init_cache(32)
        got = [o.outputs[0].token_ids for o in r.engine.generate(prompts, params)]
        assert got == want, (infer_ep, bool(mapping), rank, got, want)
        r.engine.free_cache()
        dist.barrier()


def test_rollout_rehomes_experts_over_four_ranks():
    run_distributed(_ep_rehome_worker, 4)


def _dock_worker(rank, world):
    from mindspeed_rl_b200.data.transfer_dock import GRPOTransferDock
    from mindspeed_rl_b200.runtime import rpc
    box = [None]
    if rank == 0:
        dock = GRPOTransferDock(4, 2)
        server = rpc.serve(dock)
        box[0] = server.address
    dist.broadcast_object_list(box, src=0)
    td = dock if rank == 0 else rpc.connect(box[0])
    if rank == 1:
        td.put_experience({"prompts": [torch.arange(3 + i) for i in range(8)],
                           "prompt_length": [torch.tensor([3 + i]) for i in range(8)]}, list(range(8)))
    dist.barrier()
    batch, idx = td.get_experience("actor_rollout", ["prompts", "prompt_length"], 4, get_n_samples=True)
    assert len(idx) == 4 and idx[0] % 2 == 0 and batch["prompts"].shape[0] == 4
    dist.barrier()
    assert td.all_consumed("actor_rollout")
    got = [None] * world
    dist.all_gather_object(got, sorted(idx))
    assert sorted(got[0] + got[1]) == list(range(8))      # no row handed out twice


def test_transfer_dock_over_rpc():
    run_distributed(_dock_worker, 2)


def _launch_worker(rank, world, train_tp, infer_tp):
    import os
    from mindspeed_rl_b200.config import compose
    from mindspeed_rl_b200.runtime.launch import run_rl
    cfg = compose("grpo_tiny_cpu", None, [
        f"actor_config.tensor_model_parallel_size={train_tp}",
        f"generate_config.infer_tensor_parallel_size={infer_tp}",
        f"rl_config.actor_resource.num_gpus={world}"])
    hist = run_rl(cfg, "grpo")
    if rank == 0:
        assert len(hist) == 2
        assert all(m["timing/rollout"] > 0 and "actor/pg_loss" in m for m in hist)


def _launch_disaggregated_worker(rank, world):
    """Actor on ranks 0-1 and reference model on ranks 2-3 (two data-parallel replicas each) with
    non-blocking stages: the reference forward runs on its own ranks while the actor ranks go on,
    and the update consumes the ``ref_log_prob`` column the other group wrote.  Both models start
    from the same seed, so the first update sees a KL of (almost) zero."""
    from mindspeed_rl_b200.config import compose
    from mindspeed_rl_b200.runtime.launch import run_rl
    cfg = compose("grpo_tiny_cpu", None, [
        "rl_config.use_integrated_worker=false", "rl_config.blocking=false",
        "rl_config.actor_resource.num_gpus=2", "+rl_config.reference_resource.num_gpus=2",
        "+ref_config.model=tiny_qwen2", "+ref_config.micro_batch_size=4"])
    hist = run_rl(cfg, "grpo")
    if rank == 0:
        assert len(hist) == 2
        for m in hist:
            assert m["timing/rollout"] > 0 and m["timing/reference_model"] > 0
            assert "actor/kl_loss" in m and "actor/pg_loss" in m
        assert abs(hist[0]["actor/kl_loss"]) < 1e-4, hist[0]["actor/kl_loss"]


def test_launch_grpo_disaggregated_reference_group():
    run_distributed(_launch_disaggregated_worker, 4)


def test_placement_plan():
    from mindspeed_rl_b200.config import RLConfig
    from mindspeed_rl_b200.runtime.placement import plan_placement
    co = plan_placement(8, RLConfig(dict(actor_resource={"num_gpus": 8})))
    assert co.of("reference") == list(range(8)) and not co.disjoint_roles()
    rl = RLConfig(dict(use_integrated_worker=False, actor_resource={"num_gpus": 8}, reference_resource={"num_gpus": 4},
                       critic_resource={"num_gpus": 4}))
    p = plan_placement(16, rl, gpus_per_node=8)
    assert p.of("actor") == list(range(8)) and p.of("reference") == [8, 9, 10, 11] and p.of("critic") == [12, 13, 14, 15]
    assert p.of("reward") == p.of("actor") and p.disjoint_roles() and not p.colocated("critic", "actor")
    rl = RLConfig(dict(use_integrated_worker=False, actor_resource={"num_gpus": 6}, reference_resource={"num_gpus": 4}))
    assert plan_placement(16, rl, gpus_per_node=8).of("reference") == [8, 9, 10, 11]      # not split over two nodes
    import pytest
    with pytest.raises(ValueError):
        plan_placement(8, rl, gpus_per_node=8)


def _launch_moe_ep_worker(rank, world):
    """Whole GRPO iterations of a small MoE model with expert parallelism 2: the two ranks are
    data-parallel replicas for rollout and training, exchange tokens in every MoE layer and
    therefore step their rollout engines together."""
    from mindspeed_rl_b200.config import compose
    from mindspeed_rl_b200.runtime.launch import run_rl
    cfg = compose("grpo_tiny_cpu", None, [
        "actor_config.expert_model_parallel_size=2", f"rl_config.actor_resource.num_gpus={world}",
        "+model.tiny_qwen2.num_experts=4", "+model.tiny_qwen2.moe_router_topk=2",
        "+model.tiny_qwen2.moe_ffn_hidden_size=32", "+model.tiny_qwen2.norm_topk_prob=true",
        "+model.tiny_qwen2.moe_aux_loss_coeff=0.001"])
    hist = run_rl(cfg, "grpo")
    if rank == 0:
        assert len(hist) == 2
        assert all(m["timing/rollout"] > 0 and "actor/pg_loss" in m for m in hist)


def test_launch_grpo_moe_expert_parallel():
    run_distributed(_launch_moe_ep_worker, 2)


def test_launch_grpo_tp2_rollout_tp1_reshard():
    """Full ``run_rl`` on 2 gloo ranks: training TP=2, rollout TP=1 (two rollout replicas) through
    the resharding plan's gathered fallback."""
    run_distributed(_launch_worker, 2, 2, 1)


def test_launch_grpo_dp2():
    run_distributed(_launch_worker, 2, 1, 1)


def _tp_grad_sync_worker(rank, world):
    """SP + QK-norm: replicated parameters' gradients are summed over TP by ``finish_grad_sync`` and
    the optimizer's global gradient norm counts them once."""
    from mindspeed_rl_b200.models.gpt import GPTModel, PackedMeta
    from mindspeed_rl_b200.models.transformer_config import TransformerConfig
    from mindspeed_rl_b200.optim.distributed_optimizer import DistributedOptimizer
    from mindspeed_rl_b200.parallel.ddp import DistributedDataParallel
    from mindspeed_rl_b200.parallel.state import initialize_model_parallel
    from mindspeed_rl_b200.parallel.tp_comm import TPComm
    ps = initialize_model_parallel(tensor_model_parallel_size=world)
    kw = dict(num_layers=2, hidden_size=32, ffn_hidden_size=64, num_attention_heads=4, num_query_groups=2,
              vocab_size=64, add_qkv_bias=True, qk_layernorm=True, params_dtype=torch.float32,
              max_position_embeddings=128)
    full = GPTModel(TransformerConfig(**kw), device="cpu", seed=5)
    cfg = TransformerConfig(tensor_model_parallel_size=world, sequence_parallel=True, **kw)
    comm = TPComm(ps.group("tp"), True, world_size=world, rank=rank)
    core = GPTModel(cfg, comm, device="cpu")
    core.load_state_dict(_shard_state(full.state_dict(), cfg, world, rank))
    model = DistributedDataParallel(core, None, 1)
    model.attach_tensor_parallel(ps.group("tp"), world, True)
    opt = DistributedOptimizer(model.buffers, lr=0.0, clip_grad=1e9, model_parallel_group=ps.group("tp"),
                               tp_rank=rank)
    meta = PackedMeta.from_lengths([6, 10], "cpu", align=world)
    t = int(meta.cu_seqlens[-1])
    g = torch.Generator().manual_seed(1)
    ids, labels, w = torch.randint(0, 64, (t,), generator=g), torch.randint(0, 64, (t,), generator=g), torch.randn(t, generator=g)
    (full.forward_logprob(ids, labels, meta, 1.0, False)[0] * w).sum().backward()
    (core.forward_logprob(ids, labels, meta, 1.0, False)[0] * w).sum().backward()
    model.finish_grad_sync()
    want = _shard_state({n: p.grad for n, p in full.named_parameters()}, cfg, world, rank)
    for n, p in core.named_parameters():
        assert torch.allclose(p.main_grad, want[n], atol=2e-4, rtol=1e-3), (n, (p.main_grad - want[n]).abs().max())
    full_norm = torch.sqrt(sum((p.grad.float() ** 2).sum() for p in full.parameters()))
    norm = torch.sqrt(opt.compute_grad_norm())
    assert torch.allclose(norm.reshape(()), full_norm, rtol=1e-4), (float(norm), float(full_norm))


def _mla_tp_worker(rank, world):
    """Latent attention under TP + SP: heads are split, the down-projections and their norms are
    replicated; their gradients (each rank sees its own heads only) are summed by ``finish_grad_sync``."""
    from mindspeed_rl_b200.models.gpt import GPTModel, PackedMeta
    from mindspeed_rl_b200.models.transformer_config import TransformerConfig
    from mindspeed_rl_b200.parallel.ddp import DistributedDataParallel
    from mindspeed_rl_b200.parallel.state import initialize_model_parallel
    from mindspeed_rl_b200.parallel.tp_comm import TPComm
    ps = initialize_model_parallel(tensor_model_parallel_size=world)
    kw = dict(num_layers=2, hidden_size=32, ffn_hidden_size=64, num_attention_heads=4, num_query_groups=4,
              vocab_size=64, params_dtype=torch.float32, max_position_embeddings=128, multi_latent_attention=True,
              q_lora_rank=12, kv_lora_rank=8, qk_head_dim=8, qk_pos_emb_head_dim=8, v_head_dim=8)
    full = GPTModel(TransformerConfig(**kw), device="cpu", seed=5)
    cfg = TransformerConfig(tensor_model_parallel_size=world, sequence_parallel=True, **kw)
    comm = TPComm(ps.group("tp"), True, world_size=world, rank=rank)
    core = GPTModel(cfg, comm, device="cpu")
    core.load_state_dict(_shard_state(full.state_dict(), cfg, world, rank))
    model = DistributedDataParallel(core, None, 1)
    model.attach_tensor_parallel(ps.group("tp"), world, True)
    meta = PackedMeta.from_lengths([6, 10], "cpu", align=world)
    t = int(meta.cu_seqlens[-1])
    g = torch.Generator().manual_seed(1)
    ids, labels, w = torch.randint(0, 64, (t,), generator=g), torch.randint(0, 64, (t,), generator=g), torch.randn(t, generator=g)
    ref = full.forward_logprob(ids, labels, meta, 1.0, False)[0]
    (ref * w).sum().backward()
    got = core.forward_logprob(ids, labels, meta, 1.0, False)[0]
    assert torch.allclose(got, ref, atol=1e-4), (got - ref).abs().max()
    (got * w).sum().backward()
    model.finish_grad_sync()
    want = _shard_state({n: (p.grad if p.grad is not None else p.main_grad) for n, p in full.named_parameters()},
                        cfg, world, rank)
    for n, p in core.named_parameters():
        have = p.main_grad if p.grad is None else p.main_grad + p.grad
        assert torch.allclose(have, want[n], atol=2e-4, rtol=1e-3), (n, (have - want[n]).abs().max())


def test_latent_attention_tensor_parallel_matches_single_rank():
    run_distributed(_mla_tp_worker, 2)


def test_tp_replicated_grad_sync_and_norm():
    run_distributed(_tp_grad_sync_worker, 2)


def _pp_worker(rank, world, n_micro):
    """1F1B over ``world`` stages reproduces the single-process gradients and outputs."""
    from mindspeed_rl_b200.models.gpt import GPTModel, PackedMeta
    from mindspeed_rl_b200.models.transformer_config import TransformerConfig
    from mindspeed_rl_b200.parallel.pipeline import PipelineSchedule
    from mindspeed_rl_b200.parallel.state import initialize_model_parallel
    from mindspeed_rl_b200.reshard.planner import stage_layers
    ps = initialize_model_parallel(pipeline_model_parallel_size=world)
    cfg = TransformerConfig(num_layers=4, hidden_size=32, ffn_hidden_size=64, num_attention_heads=4,
                            num_query_groups=2, vocab_size=64, add_qkv_bias=True, params_dtype=torch.float32,
                            max_position_embeddings=128)
    full = GPTModel(cfg, device="cpu", seed=5)
    layers = stage_layers(cfg.num_layers, world)[rank]
    stage = GPTModel(cfg, device="cpu", pre_process=rank == 0, post_process=rank == world - 1, layer_numbers=layers)
    sd = {}
    for k, v in full.state_dict().items():
        if k.startswith("decoder.layers."):
            idx = int(k.split(".")[2])
            if idx in layers:
                sd[f"decoder.layers.{layers.index(idx)}." + k.split(".", 3)[3]] = v
        elif k.startswith("embedding."):
            if rank == 0:
                sd[k] = v
        elif rank == world - 1:
            sd[k] = v
    stage.load_state_dict(sd)
    g = torch.Generator().manual_seed(3)
    mbs = []
    for i in range(n_micro):
        meta = PackedMeta.from_lengths([5 + i, 9], "cpu")
        t = int(meta.cu_seqlens[-1])
        mbs.append(dict(meta=meta, t=t, ids=torch.randint(0, 64, (t,), generator=g),
                        labels=torch.randint(0, 64, (t,), generator=g), w=torch.randn(t, generator=g)))
    want_lp = []
    for mb in mbs:
        lp, _ = full.forward_logprob(mb["ids"], mb["labels"], mb["meta"], 1.0, False)
        (lp * mb["w"]).sum().backward()
        want_lp.append(lp.detach())
    sched = PipelineSchedule(ps.group("pp"), rank, world, ps.get_pipeline_model_parallel_prev_rank(),
                             ps.get_pipeline_model_parallel_next_rank(), cfg.hidden_size, torch.float32, "cpu")

    def stage_fwd(mb, h_in):
        x = mb["ids"] if h_in is None else h_in
        if not stage.post_process:
            return stage.hidden_states(x, mb["meta"])
        return stage.forward_logprob(x, mb["labels"], mb["meta"], 1.0, False)

    got = []

    def last_bwd(mb, out):
        lp, _ = out
        got.append(lp.detach())
        (lp * mb["w"]).sum().backward()

    sched.forward_backward(mbs, lambda m: m["t"], stage_fwd, last_bwd)
    if rank == world - 1:
        assert len(got) == n_micro and all(torch.allclose(a, b, atol=1e-5) for a, b in zip(got, want_lp))
    full_grads = {n: p.grad for n, p in full.named_parameters()}
    for n, p in stage.named_parameters():
        if n.startswith("decoder.layers."):
            idx = layers[int(n.split(".")[2])]
            ref = full_grads[f"decoder.layers.{idx}." + n.split(".", 3)[3]]
        else:
            ref = full_grads[n]
        assert torch.allclose(p.grad, ref, atol=2e-5, rtol=1e-4), (n, (p.grad - ref).abs().max())
    with torch.no_grad():
        outs = sched.forward_only(mbs, lambda m: m["t"], stage_fwd)
    if rank == world - 1:
        assert all(torch.allclose(o[0], b, atol=1e-5) for o, b in zip(outs, want_lp))


def _vpp_worker(rank, world, n_micro, vpp, noop):
    """Interleaved (virtual-stage) schedule with an empty layer slot: gradients and outputs of the
    single-process model."""
    from mindspeed_rl_b200.models.gpt import GPTModel, PackedMeta
    from mindspeed_rl_b200.models.transformer_config import TransformerConfig
    from mindspeed_rl_b200.parallel.pipeline import PipelineSchedule
    from mindspeed_rl_b200.parallel.state import initialize_model_parallel
    from mindspeed_rl_b200.reshard.planner import stage_chunks
    ps = initialize_model_parallel(pipeline_model_parallel_size=world)
    slots = world * vpp * 2
    chunks = stage_chunks(slots, world, None, vpp, noop)[rank]
    layers = sum(chunks, [])
    n_real = slots - len(noop)
    cfg = TransformerConfig(num_layers=n_real, hidden_size=32, ffn_hidden_size=64, num_attention_heads=4,
                            num_query_groups=2, vocab_size=64, add_qkv_bias=True, params_dtype=torch.float32,
                            max_position_embeddings=128)
    full = GPTModel(cfg, device="cpu", seed=5)
    stage = GPTModel(cfg, device="cpu", pre_process=rank == 0, post_process=rank == world - 1, layer_numbers=layers,
                     chunk_sizes=[len(c) for c in chunks])
    sd = {}
    for k, v in full.state_dict().items():
        if k.startswith("decoder.layers."):
            idx = int(k.split(".")[2])
            if idx in layers:
                sd[f"decoder.layers.{layers.index(idx)}." + k.split(".", 3)[3]] = v
        elif k.startswith("embedding."):
            if rank == 0:
                sd[k] = v
        elif rank == world - 1:
            sd[k] = v
    stage.load_state_dict(sd)
    g = torch.Generator().manual_seed(3)
    mbs = []
    for i in range(n_micro):
        meta = PackedMeta.from_lengths([5 + i, 9], "cpu")
        t = int(meta.cu_seqlens[-1])
        mbs.append(dict(meta=meta, t=t, ids=torch.randint(0, 64, (t,), generator=g),
                        labels=torch.randint(0, 64, (t,), generator=g), w=torch.randn(t, generator=g)))
    want_lp = []
    for mb in mbs:
        lp, _ = full.forward_logprob(mb["ids"], mb["labels"], mb["meta"], 1.0, False)
        (lp * mb["w"]).sum().backward()
        want_lp.append(lp.detach())
    sched = PipelineSchedule(ps.group("pp"), rank, world, ps.get_pipeline_model_parallel_prev_rank(),
                             ps.get_pipeline_model_parallel_next_rank(), cfg.hidden_size, torch.float32, "cpu",
                             num_chunks=vpp, grad_group=ps.group("pp_grad"))

    def stage_fwd(mb, h_in, chunk):
        x = mb["ids"] if h_in is None else h_in
        if not stage.is_last_chunk(chunk):
            return stage.hidden_states(x, mb["meta"], chunk)
        return stage.forward_logprob(x, mb["labels"], mb["meta"], 1.0, False, chunk)

    got = {}

    def last_bwd(mb, out):
        lp, _ = out
        got[id(mb)] = lp.detach()
        (lp * mb["w"]).sum().backward()

    sched.forward_backward(mbs, lambda m: m["t"], stage_fwd, last_bwd)
    if rank == world - 1:
        assert len(got) == n_micro and all(torch.allclose(got[id(m)], b, atol=1e-5) for m, b in zip(mbs, want_lp))
    full_grads = {n: p.grad for n, p in full.named_parameters()}
    for n, p in stage.named_parameters():
        if n.startswith("decoder.layers."):
            idx = layers[int(n.split(".")[2])]
            ref = full_grads[f"decoder.layers.{idx}." + n.split(".", 3)[3]]
        else:
            ref = full_grads[n]
        assert torch.allclose(p.grad, ref, atol=2e-5, rtol=1e-4), (n, (p.grad - ref).abs().max())
    with torch.no_grad():
        outs = sched.forward_only(mbs, lambda m: m["t"], stage_fwd)
    if rank == world - 1:
        assert all(torch.allclose(o[0], b, atol=1e-5) for o, b in zip(outs, want_lp))


def test_interleaved_pipeline_matches_single_process():
    from mindspeed_rl_b200.reshard.planner import stage_chunks
    # 8 slots on 2 stages x 2 chunks, slot 7 empty: stage 0 holds layers [0,1 | 4,5], stage 1 [2,3 | 6]
    assert stage_chunks(8, 2, None, 2, [7]) == [[[0, 1], [4, 5]], [[2, 3], [6]]]
    run_distributed(_vpp_worker, 2, 4, 2, [7])        # two groups of micro-batches: warm-up, steady state, cool-down
    run_distributed(_vpp_worker, 2, 2, 2, [])         # micro-batches == stages: all forwards, then all backwards
    run_distributed(_vpp_worker, 3, 6, 2, [3])        # three stages


def test_pipeline_1f1b_matches_single_process():
    run_distributed(_pp_worker, 2, 3)
    run_distributed(_pp_worker, 4, 6)
    run_distributed(_pp_worker, 4, 2)        # fewer micro-batches than stages


def _cp_worker(rank, world, algo, ring=False, ulysses=1):
    """Context parallel (zig-zag or contiguous split, head-parallel or ring attention) == single process."""
    import os
    os.environ["MSRL_CP_RING"] = "1" if ring else "0"
    from mindspeed_rl_b200.models.gpt import GPTModel, PackedMeta
    from mindspeed_rl_b200.models.transformer_config import TransformerConfig
    from mindspeed_rl_b200.parallel.context_parallel import ContextParallel
    from mindspeed_rl_b200.parallel.state import initialize_model_parallel
    ps = initialize_model_parallel(context_parallel_size=world)
    cfg = TransformerConfig(num_layers=2, hidden_size=32, ffn_hidden_size=64, num_attention_heads=4,
                            num_query_groups=2, vocab_size=64, add_qkv_bias=True, params_dtype=torch.float32,
                            max_position_embeddings=128)
    full = GPTModel(cfg, device="cpu", seed=5)
    model = GPTModel(cfg, device="cpu", seed=5)
    meta = PackedMeta.from_lengths([6, 13, 4], "cpu", align=2 * world)
    t = int(meta.cu_seqlens[-1])
    g = torch.Generator().manual_seed(1)
    ids, labels, w = torch.randint(0, 64, (t,), generator=g), torch.randint(0, 64, (t,), generator=g), torch.randn(t, generator=g)
    ref_lp, _ = full.forward_logprob(ids, labels, meta, 1.0, False)
    (ref_lp * w).sum().backward()
    cp = ContextParallel(ps.group("cp"), world, rank, algo, meta.cu_seqlens.to(torch.int64), "cpu",
                         ulysses_degree=ulysses)
    assert cp.local_index.numel() == t // world
    if algo != "hybrid_cp_algo":
        assert cp.use_ring(model.decoder.layers[0].self_attention.layout) == (ring or world == 3)
    m_local = PackedMeta(cp.cu_local, cp.max_local, cp.take_local(meta.positions), cp=cp)
    lp_l, _ = model.forward_logprob(cp.take_local(ids), cp.take_local(labels), m_local, 1.0, False)
    lp = cp.gather_tokens(lp_l)
    assert torch.allclose(lp, ref_lp, atol=1e-5), (lp - ref_lp).abs().max()
    (lp * w).sum().backward()
    for (n, p), q in zip(model.named_parameters(), full.parameters()):
        gr = p.grad.clone()
        dist.all_reduce(gr)
        assert torch.allclose(gr / world, q.grad, atol=2e-5, rtol=1e-4), (n, (gr / world - q.grad).abs().max())


def test_context_parallel_matches_single_process():
    run_distributed(_cp_worker, 2, "megatron_cp_algo")
    run_distributed(_cp_worker, 2, "ulysses_cp_algo")


def test_hybrid_context_parallel_matches_single_process():
    run_distributed(_cp_worker, 4, "hybrid_cp_algo", False, 2)      # 2 ring positions x 2 ulysses ranks


def test_ring_attention_matches_single_process():
    run_distributed(_cp_worker, 2, "megatron_cp_algo", True)
    run_distributed(_cp_worker, 3, "megatron_cp_algo")       # 4 / 2 heads do not divide by 3: ring


def _lora_tp_worker(rank, world, sp):
    """LoRA under TP (+SP): adapters sharded like their base weights reproduce the single-process
    outputs and adapter gradients."""
    from mindspeed_rl_b200.checkpoint import convert as C
    from mindspeed_rl_b200.models import lora
    from mindspeed_rl_b200.models.gpt import GPTModel, PackedMeta
    from mindspeed_rl_b200.models.transformer_config import TransformerConfig
    from mindspeed_rl_b200.parallel.ddp import DistributedDataParallel
    from mindspeed_rl_b200.parallel.state import initialize_model_parallel
    from mindspeed_rl_b200.parallel.tp_comm import TPComm
    ps = initialize_model_parallel(tensor_model_parallel_size=world)
    targets = ("linear_qkv", "linear_proj", "linear_fc1", "linear_fc2")
    kw = dict(num_layers=2, hidden_size=32, ffn_hidden_size=64, num_attention_heads=4, num_query_groups=2,
              vocab_size=64, add_qkv_bias=True, params_dtype=torch.float32, max_position_embeddings=128,
              lora_r=4, lora_alpha=8, lora_target_modules=targets)
    full = GPTModel(TransformerConfig(**kw), device="cpu", seed=5)
    g = torch.Generator().manual_seed(3)
    for h in lora.holders(full):
        h.lora_B.data.normal_(0, 0.1, generator=g)
    cfg = TransformerConfig(tensor_model_parallel_size=world, sequence_parallel=sp, **kw)
    comm = TPComm(ps.group("tp"), sp, world_size=world, rank=rank)
    core = GPTModel(cfg, comm, device="cpu")

    def shard(state):
        out = _shard_state({k: v for k, v in state.items() if "lora_" not in k}, cfg, world, rank)
        for k, v in state.items():
            if k.endswith("linear_qkv.lora_B"):
                out[k] = C.shard_qkv(v, cfg.num_query_groups, world, rank)
            elif k.endswith("linear_fc1.lora_B"):
                gate, up = v.chunk(2, 0)
                out[k] = C.shard_fc1(gate, up, world, rank)
            elif k.endswith(("linear_proj.lora_A", "linear_fc2.lora_A")):
                out[k] = C.shard_cols(v, world, rank)
            elif "lora_" in k:
                out[k] = v.clone()
        return out

    core.load_state_dict(shard(full.state_dict()))
    model = DistributedDataParallel(core, None, 1)
    model.attach_tensor_parallel(ps.group("tp"), world, sp)
    meta = PackedMeta.from_lengths([6, 10], "cpu", align=world)
    t = int(meta.cu_seqlens[-1])
    ids, labels, w = torch.randint(0, 64, (t,), generator=g), torch.randint(0, 64, (t,), generator=g), torch.randn(t, generator=g)
    ref_lp, _ = full.forward_logprob(ids, labels, meta, 1.0, False)
    (ref_lp * w).sum().backward()
    lp, _ = core.forward_logprob(ids, labels, meta, 1.0, False)
    (lp * w).sum().backward()
    model.finish_grad_sync()
    assert torch.allclose(lp, ref_lp, atol=1e-4), (lp - ref_lp).abs().max()
    want = shard({n: p.grad for n, p in full.named_parameters() if p.grad is not None})
    checked = 0
    for n, p in core.named_parameters():
        if p.requires_grad:
            assert torch.allclose(p.main_grad, want[n], atol=2e-4, rtol=1e-3), (n, (p.main_grad - want[n]).abs().max())
            checked += 1
    assert checked == 2 * 4 * 2
    # rollout at another TP size: the frozen base weights and the adapters travel through the reshard plan and
    # the rollout copy holds W + (alpha / r) B A of the whole model
    from mindspeed_rl_b200.reshard.planner import Resharder
    from mindspeed_rl_b200.rollout.engine import LLMEngine

    again = DistributedDataParallel(core, None, 1, frozen_buffer=True)
    assert again.frozen_buffer is not None and len(again.frozen_buffer.params) > 0
    r = Resharder(cfg, again, ps, 1, "cpu", lambda icfg, c: LLMEngine(icfg, "cpu", max_num_seqs=2, max_model_len=32,
                                                                      block_size=4))
    rw = r.reshard(core)
    for li, layer in enumerate(full.decoder.layers):
        for got, holder in ((rw.layers[li].qkv_w, layer.self_attention.linear_qkv),
                            (rw.layers[li].o_w, layer.self_attention.linear_proj),
                            (rw.layers[li].gate_up_w, layer.mlp.linear_fc1), (rw.layers[li].down_w, layer.mlp.linear_fc2)):
            assert torch.allclose(got, lora.merged_weight(holder), atol=1e-5), (li, (got - lora.merged_weight(holder)).abs().max())


def test_lora_tensor_parallel_matches_single_rank():
    run_distributed(_lora_tp_worker, 2, False)
    run_distributed(_lora_tp_worker, 2, True)


def _launch_pp_worker(rank, world):
    from mindspeed_rl_b200.config import compose
    from mindspeed_rl_b200.runtime.launch import run_rl
    cfg = compose("grpo_tiny_cpu", None, [
        "actor_config.pipeline_model_parallel_size=2", "actor_config.no_pad_to_seq_lengths=true",
        "generate_config.infer_tensor_parallel_size=1",
        "megatron_training.train_iters=1", f"rl_config.actor_resource.num_gpus={world}"])
    hist = run_rl(cfg, "grpo")
    if rank == 0:
        assert len(hist) == 1 and "actor/pg_loss" in hist[0] and hist[0]["timing/update"] > 0


def test_launch_grpo_pp2():
    """GRPO with a 2-stage pipeline for training and a full-depth rollout replica per rank."""
    run_distributed(_launch_pp_worker, 2)


def _launch_vpp_worker(rank, world):
    """GRPO with an interleaved pipeline (2 stages x 2 chunks over 4 layer slots, one of them empty):
    training through virtual stages, then the 3 real layers gathered into a full-depth rollout replica."""
    from mindspeed_rl_b200.config import compose
    from mindspeed_rl_b200.runtime.launch import run_rl
    cfg = compose("grpo_tiny_cpu", None, [
        "actor_config.pipeline_model_parallel_size=2", "actor_config.no_pad_to_seq_lengths=true",
        "+actor_config.num_layers_per_virtual_pipeline_stage=1", "+actor_config.noop_layers=3",
        "+model.tiny_qwen2.num_layers=4", "generate_config.infer_tensor_parallel_size=1",
        "megatron_training.train_iters=2", f"rl_config.actor_resource.num_gpus={world}"])
    hist = run_rl(cfg, "grpo")
    if rank == 0:
        assert len(hist) == 2 and all("actor/pg_loss" in m and m["timing/update"] > 0 for m in hist)
        assert abs(hist[0]["actor/kl_loss"]) < 1e-4


def test_launch_grpo_interleaved_pipeline_with_empty_slot():
    run_distributed(_launch_vpp_worker, 2)


def _pairwise_batch(pairs=4, seq=12, vocab=96, seed=0):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(1, vocab, (2 * pairs, seq), generator=g)
    lens = torch.randint(6, seq + 1, (2 * pairs,), generator=g)
    mask = (torch.arange(seq).unsqueeze(0) < lens.unsqueeze(1)).long()
    labels = torch.where((torch.arange(seq).unsqueeze(0) >= 3) & (mask > 0), ids, torch.full_like(ids, -100))
    return {"input_ids": ids * mask, "attention_mask": mask, "labels": labels}


def _dpo_build(ps, world, rank):
    from mindspeed_rl_b200.models.gpt import GPTModel
    from mindspeed_rl_b200.models.transformer_config import TransformerConfig
    from mindspeed_rl_b200.optim.distributed_optimizer import DistributedOptimizer
    from mindspeed_rl_b200.parallel.ddp import DistributedDataParallel
    from mindspeed_rl_b200.trainer.dpo_trainer import DPOTrainer
    cfg = TransformerConfig(num_layers=2, hidden_size=32, ffn_hidden_size=64, num_attention_heads=4, num_query_groups=2,
                            vocab_size=96, params_dtype=torch.float32, max_position_embeddings=64)
    core = GPTModel(cfg, device="cpu", seed=11)
    ref = GPTModel(cfg, device="cpu", seed=12)
    for p in ref.parameters():
        p.requires_grad_(False)
    group = ps.group("dp_cp") if ps is not None else None
    model = DistributedDataParallel(core, group, world)
    opt = DistributedOptimizer(model.buffers, lr=1e-3, betas=(0.9, 0.95), weight_decay=0.0, clip_grad=1.0,
                               dp_group=group, dp_rank=rank)
    return core, DPOTrainer(model, ref, opt, beta=0.5, train_iters=2, device="cpu", dp_group=group, dp_rank=rank,
                            dp_size=world)


def _dpo_dp_worker(rank, world, want):
    from mindspeed_rl_b200.parallel.state import initialize_model_parallel
    ps = initialize_model_parallel()
    core, trainer = _dpo_build(ps, world, rank)
    hist = trainer.train(iter([_pairwise_batch(seed=s) for s in range(2)]))
    for got, ref in zip(hist, want["hist"]):
        for k in ("dpo/loss", "dpo/margin", "dpo/accuracy", "grad_norm"):
            assert abs(got[k] - ref[k]) < 1e-5 * max(1.0, abs(ref[k])), (k, got[k], ref[k])
        assert got["samples_per_sec"] > 0
    # Adam turns a rounding-level difference of a near-zero gradient into a step of lr, so single elements may
    # sit one step apart; on average the two runs coincide
    for n, p in core.named_parameters():
        d = (p - want["params"][n]).abs()
        assert float(d.mean()) < 2e-6 and float(d.max()) < 2.5e-3, (n, float(d.mean()), float(d.max()))


def test_dpo_data_parallel_matches_single_rank():
    """Two replicas that each train on half of the pairs end where one rank with all pairs ends, and report
    the same loss, margin, accuracy and gradient norm."""
    core, trainer = _dpo_build(None, 1, 0)
    hist = trainer.train(iter([_pairwise_batch(seed=s) for s in range(2)]))
    assert hist[0]["dpo/loss"] > 0 and hist[0]["grad_norm"] > 0
    want = {"hist": [{k: v for k, v in h.items()} for h in hist],
            "params": {n: p.detach().clone() for n, p in core.named_parameters()}}
    run_distributed(_dpo_dp_worker, 2, want)


def _launch_cp_worker(rank, world, algo):
    """Whole GRPO iterations with the training side context-parallel over both ranks (every sequence's tokens are
    split between them in the log-prob passes and the update), rollout replicas per rank."""
    from mindspeed_rl_b200.config import compose
    from mindspeed_rl_b200.runtime.launch import run_rl
    cfg = compose("grpo_tiny_cpu", None, [
        "actor_config.context_parallel_size=2", f"actor_config.context_parallel_algo={algo}",
        f"rl_config.actor_resource.num_gpus={world}", "megatron_training.global_batch_size=4",
        "rl_config.mini_batch_size=4", "rl_config.n_samples_per_prompt=2",
        "generate_config.sampling_config.max_tokens=8", "megatron_training.train_iters=2"])
    hist = run_rl(cfg, "grpo")
    if rank == 0:
        assert len(hist) == 2
        for m in hist:
            assert m["timing/rollout"] > 0 and "actor/pg_loss" in m and m["actor/grad_norm"] >= 0
        # old and reference log-probs come from the same weights in iteration 1: a context-parallel pass that
        # mixed up token order would show up as a KL far from zero
        assert abs(hist[0]["actor/kl_loss"]) < 1e-4 and abs(hist[0]["actor/ppo_kl"]) < 1e-4


def test_launch_grpo_context_parallel_ring():
    run_distributed(_launch_cp_worker, 2, "megatron_cp_algo")


def test_launch_grpo_context_parallel_all_to_all():
    run_distributed(_launch_cp_worker, 2, "ulysses_cp_algo")


def _launch_overlap_worker(rank, world, want):
    """Two data-parallel replicas with bucketed gradient reduction behind the backward and the parameter gather
    pipelined behind the optimizer's chunks: same numbers as the plain schedule."""
    from mindspeed_rl_b200.config import compose
    from mindspeed_rl_b200.runtime.launch import run_rl
    cfg = compose("grpo_tiny_cpu", None, [
        f"rl_config.actor_resource.num_gpus={world}", "megatron_training.global_batch_size=4",
        "rl_config.mini_batch_size=4", "rl_config.n_samples_per_prompt=4", "actor_config.lr=1e-3",
        "generate_config.sampling_config.max_tokens=48", "megatron_training.train_iters=2"] +
        (["actor_config.overlap_grad_reduce=true", "actor_config.overlap_param_gather=true"] if want is not None else []))
    hist = run_rl(cfg, "grpo")
    if rank == 0:
        got = [(m["actor/grad_norm"], m["actor/entropy"], m["response_length/mean"]) for m in hist]
        if want is None:
            import json, os
            with open(os.environ["MSRL_TEST_OUT"], "w") as fh:
                json.dump(got, fh)
        else:
            for a, b in zip(got, want):
                assert all(abs(x - y) <= 1e-5 * max(1.0, abs(y)) for x, y in zip(a, b)), (got, want)


def test_launch_grpo_dp2_with_overlapped_collectives(tmp_path, monkeypatch):
    import json
    monkeypatch.setenv("MSRL_TEST_OUT", str(tmp_path / "plain.json"))
    run_distributed(_launch_overlap_worker, 2, None)
    want = json.loads((tmp_path / "plain.json").read_text())
    assert len(want) == 2 and want[0][0] > 0
    run_distributed(_launch_overlap_worker, 2, want)


def _launch_reward_model_worker(rank, world):
    """Actor on rank 0, reference model on rank 1, a model-based reward scorer (decoder + scalar head) on rank 2:
    the scores column is written by the scorer's group and consumed by the advantage stage."""
    from mindspeed_rl_b200.config import compose
    from mindspeed_rl_b200.runtime.launch import run_rl
    cfg = compose("grpo_tiny_cpu", None, [
        "rl_config.use_integrated_worker=false", "rl_config.actor_resource.num_gpus=1",
        "+rl_config.reference_resource.num_gpus=1", "+rl_config.reward_resource.num_gpus=1", "+reward_config.model=tiny_qwen2", "+reward_config.micro_batch_size=4",
        "+ref_config.model=tiny_qwen2", "+ref_config.micro_batch_size=4", "+rl_config.rule_reward=false",
        "megatron_training.global_batch_size=4", "rl_config.mini_batch_size=4", "rl_config.n_samples_per_prompt=2",
        "generate_config.sampling_config.max_tokens=8", "megatron_training.train_iters=2"])
    hist = run_rl(cfg, "grpo")
    if rank == 0:
        assert len(hist) == 2
        for m in hist:
            assert m["timing/reward_model"] > 0 and "actor/pg_loss" in m
            assert m["grpo/score/max"] != m["grpo/score/min"]            # a random scalar head: scores differ
            assert m["actor/grad_norm"] > 0


def test_launch_grpo_reward_model_on_its_own_rank():
    run_distributed(_launch_reward_model_worker, 3)


def _launch_critic_rank_worker(rank, world, blocking):
    """PPO with the actor (and its reference) on rank 0 and the critic on rank 1: value estimates, advantages and
    both updates flow through the experience store served by the driver."""
    from mindspeed_rl_b200.config import compose
    from mindspeed_rl_b200.runtime.launch import run_rl
    cfg = compose("grpo_tiny_cpu", None, [
        "rl_config.actor_resource.num_gpus=1", "megatron_training.stage=ray_ppo", "rl_config.adv_estimator=gae",
        "+critic_config.model=tiny_qwen2", "+critic_config.micro_batch_size=4", "+critic_config.lr=1e-5",
        "+rl_config.critic_resource.num_gpus=1", "megatron_training.global_batch_size=4", "rl_config.mini_batch_size=4",
        "rl_config.n_samples_per_prompt=2", "generate_config.sampling_config.max_tokens=8",
        "megatron_training.train_iters=2", f"rl_config.blocking={'true' if blocking else 'false'}"])
    hist = run_rl(cfg, "ppo")
    if rank == 0:
        assert len(hist) == 2
        assert all(m["critic/vf_loss"] >= 0 and m["timing/update_critic"] > 0 and m["timing/critic_model"] > 0
                   and "actor/pg_loss" in m for m in hist)


def test_launch_ppo_critic_on_its_own_rank():
    run_distributed(_launch_critic_rank_worker, 2, True, timeout=240)
    run_distributed(_launch_critic_rank_worker, 2, False, timeout=240)


def _launch_partial_rollout_worker(rank, world):
    """Partial rollout over two data-parallel replicas: when more prompt groups than one training batch have
    completed, every stage (rewards, log-probs, advantages, update) works on the same first groups, so the two
    replicas get equal shares and the update's collectives line up."""
    from mindspeed_rl_b200.config import compose
    from mindspeed_rl_b200.runtime.launch import run_rl
    cfg = compose("grpo_tiny_cpu", None, [
        f"rl_config.actor_resource.num_gpus={world}", "megatron_training.global_batch_size=4",
        "rl_config.mini_batch_size=4", "rl_config.n_samples_per_prompt=2", "rl_config.partial_rollout_max_split=2",
        "generate_config.sampling_config.max_tokens=16", "megatron_training.train_iters=3"])
    hist = run_rl(cfg, "grpo")
    if rank == 0:
        assert len(hist) == 3
        assert all(m["response_length/max"] <= 16 and "actor/pg_loss" in m for m in hist)


def test_launch_grpo_partial_rollout_dp2():
    run_distributed(_launch_partial_rollout_worker, 2, timeout=240)


def _launch_misc_worker(rank, world, overrides, expect_key):
    from mindspeed_rl_b200.config import compose
    from mindspeed_rl_b200.runtime.launch import run_rl
    cfg = compose("grpo_tiny_cpu", None, [
        f"rl_config.actor_resource.num_gpus={world}", "megatron_training.global_batch_size=4",
        "rl_config.mini_batch_size=4", "rl_config.n_samples_per_prompt=2",
        "generate_config.sampling_config.max_tokens=8", "megatron_training.train_iters=2"] + list(overrides))
    hist = run_rl(cfg, "grpo")
    if rank == 0:
        assert len(hist) == 2 and all(expect_key in m and "actor/pg_loss" in m for m in hist)


def test_launch_grpo_multi_turn_with_tensor_parallel_rollout():
    """The multi-turn loop with the tool file of the shipped recipe on a TP2 rollout group (the ranks of the
    group step the loop together); the whitespace tokenizer never produces a call, so no tool runs."""
    run_distributed(_launch_misc_worker, 2, [
        "rl_config.multi_turn_enable=true", "rl_config.async_engine=true",
        "rl_config.tool_config_path=" + os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "configs",
                                                      "tools", "retool.yaml"), "rl_config.max_tool_calls=1",
        "rl_config.max_parallel_calls=1", "rl_config.max_total_response_length=64",
        "rl_config.max_tool_response_length=16", "rl_config.tool_parser_format=hermes",
        "actor_config.tensor_model_parallel_size=2", "generate_config.infer_tensor_parallel_size=2"],
        "tool_call_num/mean", timeout=240)


def test_launch_grpo_vision_stage_on_its_own_rank(tmp_path):
    import json
    import numpy as np
    rng = np.random.default_rng(0)
    with open(tmp_path / "rows.jsonl", "w") as f:
        for i in range(8):
            img = (rng.random((28, 42, 3)) * 255).astype(np.uint8).tolist()
            f.write(json.dumps({"prompt": f"5 6 <image> 7 {8 + i}", "images": [img], "answer": str(i)}) + "\n")
    run_distributed(_launch_misc_worker, 2, [
        "rl_config.actor_resource.num_gpus=1", "+rl_config.vit_resource.num_gpus=1",
        f"megatron_training.data_path={tmp_path / 'rows.jsonl'}", "+rl_config.is_multimodal=true",
        "+rl_config.reuse_image_embeds=true", "generate_config.enable_prefix_caching=false",
        "rl_config.use_remove_padding=false", "+megatron_training.image_token_id=1000",
        "+megatron_training.vision_start_token_id=1001", "+megatron_training.vision_end_token_id=1002",
        "+vit_config.hidden_size=32", "+vit_config.num_layers=1", "+vit_config.num_attention_heads=2",
        "+vit_config.ffn_hidden_size=48", "+rl_config.max_prompt_length=96"], "timing/vit_image_emb", timeout=240)


def _moe_tp_worker(rank, world, sp, extend):
    """Expert layers under tensor parallelism against the single-rank model: experts replicated over the TP ranks
    (with and without sequence parallelism) or spread over them (``moe_tp_extend_ep``); one shared expert."""
    from mindspeed_rl_b200.models.gpt import GPTModel, PackedMeta
    from mindspeed_rl_b200.models.transformer_config import TransformerConfig
    from mindspeed_rl_b200.parallel.state import initialize_model_parallel, set_parallel_state
    from mindspeed_rl_b200.parallel.tp_comm import TPComm
    kw = dict(num_layers=2, hidden_size=32, ffn_hidden_size=64, num_attention_heads=4, num_query_groups=2,
              vocab_size=64, add_qkv_bias=True, params_dtype=torch.float32, max_position_embeddings=128,
              num_experts=4, moe_router_topk=2, moe_ffn_hidden_size=16, n_shared_experts=1, moe_aux_loss_coeff=0.01)
    if sp:
        # under sequence parallelism the balancing loss is computed per token shard (every TP rank balances its own
        # tokens), which is not the single-rank loss over all tokens: it stays out of the strict comparison
        kw["moe_aux_loss_coeff"] = 0.0
    set_parallel_state(None)
    initialize_model_parallel(world_size=1, rank=0)          # the reference model holds every expert
    torch.manual_seed(0)
    full = GPTModel(TransformerConfig(**kw), device="cpu", seed=5)
    set_parallel_state(None)
    ps = initialize_model_parallel(tensor_model_parallel_size=world, moe_tp_extend_ep=extend)
    cfg = TransformerConfig(tensor_model_parallel_size=world, sequence_parallel=sp, **kw)
    comm = TPComm(ps.group("tp"), sp, world_size=world, rank=rank)
    model = GPTModel(cfg, comm, device="cpu")
    ep = ps.size("ep")
    assert ep == (world if extend else 1)
    h, f, e = 32, 16, 4
    per = e // ep
    er = ps.rank_in("ep")

    def shard(state):
        out = _shard_state(state, cfg, world, rank)
        for k, v in state.items():
            if k.endswith("experts.weight1"):
                out[k] = v.view(h, e, 2 * f)[:, er * per:(er + 1) * per].reshape(h, -1).contiguous()
            elif k.endswith("experts.weight2"):
                out[k] = v.view(e, f, h)[er * per:(er + 1) * per].reshape(-1, h).contiguous()
            elif "shared_experts.linear_fc1" in k or "shared_experts.linear_fc2" in k:
                pass                                        # cut like the dense MLP by _shard_state
            elif ".mlp.router." in k:
                out[k] = v.clone()
        return out

    model.load_state_dict(shard(full.state_dict()))
    lens = [6, 10]
    meta = PackedMeta.from_lengths(lens, "cpu", align=world)
    t = int(meta.cu_seqlens[-1])
    g = torch.Generator().manual_seed(1)
    ids, labels, w = torch.randint(0, 64, (t,), generator=g), torch.randint(0, 64, (t,), generator=g), torch.randn(t, generator=g)
    ref_lp, ref_ent = full.forward_logprob(ids, labels, meta, 0.9, True)
    (ref_lp * w + 0.1 * ref_ent).sum().backward()
    if sp:
        model.embed = lambda x, _m=model: _seq_shard(_orig_embed(_m, x), world, rank)
    lp, ent = model.forward_logprob(ids, labels, meta, 0.9, True)
    (lp * w + 0.1 * ent).sum().backward()
    assert torch.allclose(lp, ref_lp, atol=1e-4), (lp - ref_lp).abs().max()
    assert torch.allclose(ent, ref_ent, atol=1e-4)
    want = shard({n: p.grad for n, p in full.named_parameters()})
    bad = []
    for n, p in model.named_parameters():
        g_ = p.grad
        partial = sp and ((p.dim() == 1 and "linear_qkv" not in n) or n.endswith("router.weight")
                          or (".experts." in n and not extend))
        assert bool(getattr(p, "tp_reduce_grad", False)) == (sp and ".experts." in n and not extend), n
        if partial:                                          # what the gradient sync adds up over TP
            dist.all_reduce(g_)
        if not torch.allclose(g_, want[n], atol=3e-4, rtol=2e-3):
            bad.append((n, float((g_ - want[n]).abs().max()), float(want[n].abs().max())))
    assert not bad, bad


def test_expert_layers_under_tensor_parallelism_match_single_rank():
    run_distributed(_moe_tp_worker, 2, False, False, timeout=240)     # experts replicated, tokens replicated
    run_distributed(_moe_tp_worker, 2, True, False, timeout=240)      # experts replicated, tokens split over TP
    run_distributed(_moe_tp_worker, 2, True, True, timeout=240)       # experts spread over the TP ranks


def test_launch_grpo_expert_recipe_shape():
    """The 30B-A3B recipe's layout scaled down to 4 ranks: training TP2 x EP2 with the experts spread over
    TP x EP and sequence parallelism, rollout TP1 x EP4 (dense weights gathered over TP, experts re-homed)."""
    run_distributed(_launch_misc_worker, 4, [
        "actor_config.tensor_model_parallel_size=2", "actor_config.expert_model_parallel_size=2",
        "+actor_config.moe_tp_extend_ep=true", "+actor_config.sequence_parallel=true",
        "generate_config.infer_tensor_parallel_size=1", "generate_config.infer_expert_parallel_size=4",
        "+model.tiny_qwen2.num_experts=4", "+model.tiny_qwen2.moe_router_topk=2",
        "+model.tiny_qwen2.moe_ffn_hidden_size=32", "+model.tiny_qwen2.norm_topk_prob=true",
        "generate_config.sampling_config.max_tokens=32"], "actor/grad_norm", timeout=280)


def test_launch_grpo_latent_attention_expert_recipe_shape():
    """The 671B recipe's structure scaled down to 4 ranks: latent attention, a dense first layer, sigmoid-routed
    experts with a shared expert, training TP2 x PP2 with the experts spread over TP and sequence parallelism,
    rollout TP2 x EP2 through the resharding plan."""
    run_distributed(_launch_misc_worker, 4, [
        "+model.tiny_qwen2.multi_latent_attention=true", "+model.tiny_qwen2.q_lora_rank=48",
        "+model.tiny_qwen2.kv_lora_rank=32", "+model.tiny_qwen2.qk_head_dim=32",
        "+model.tiny_qwen2.qk_pos_emb_head_dim=32", "+model.tiny_qwen2.v_head_dim=64",
        "+model.tiny_qwen2.group_query_attention=false", "+model.tiny_qwen2.add_qkv_bias=false",
        "+model.tiny_qwen2.num_experts=4", "+model.tiny_qwen2.moe_router_topk=2",
        "+model.tiny_qwen2.moe_ffn_hidden_size=32", "+model.tiny_qwen2.n_shared_experts=1",
        "+model.tiny_qwen2.first_k_dense_replace=1", "+model.tiny_qwen2.moe_router_score_function=sigmoid",
        "+model.tiny_qwen2.norm_topk_prob=true", "actor_config.tensor_model_parallel_size=2",
        "actor_config.pipeline_model_parallel_size=2", "+actor_config.moe_tp_extend_ep=true",
        "+actor_config.sequence_parallel=true", "+actor_config.no_pad_to_seq_lengths=true",
        "generate_config.infer_tensor_parallel_size=2", "generate_config.infer_expert_parallel_size=2",
        "generate_config.sampling_config.max_tokens=16"], "actor/grad_norm", timeout=280)


def test_launch_grpo_lora_recipe_shape():
    """The LoRA recipe's layout scaled down to 4 ranks: training TP2 x PP2 with sequence parallelism, adapters on
    all four linears, rollout TP2 with the adapters carried through the resharding plan and folded there."""
    run_distributed(_launch_misc_worker, 4, [
        "actor_config.tensor_model_parallel_size=2", "actor_config.pipeline_model_parallel_size=2",
        "generate_config.infer_tensor_parallel_size=2", "+actor_config.no_pad_to_seq_lengths=true",
        "+actor_config.sequence_parallel=true", "+actor_config.lora_r=4", "+actor_config.lora_alpha=8",
        "+actor_config.lora_target_modules=[linear_qkv,linear_proj,linear_fc1,linear_fc2]",
        "generate_config.sampling_config.max_tokens=32", "actor_config.lr=1e-3"], "actor/grad_norm", timeout=280)


def _launch_dapo_long_context_worker(rank, world):
    from mindspeed_rl_b200.config import compose
    from mindspeed_rl_b200.runtime.launch import run_rl
    cfg = compose("grpo_tiny_cpu", None, [
        f"rl_config.actor_resource.num_gpus={world}", "megatron_training.stage=ray_dapo",
        "actor_config.tensor_model_parallel_size=2", "actor_config.pipeline_model_parallel_size=2",
        "actor_config.context_parallel_size=2", "actor_config.context_parallel_algo=megatron_cp_algo",
        "generate_config.infer_tensor_parallel_size=1", "+actor_config.no_pad_to_seq_lengths=true",
        "+actor_config.sequence_parallel=true", "+rl_config.use_dynamic_bsz=true",
        "+rl_config.max_packing_token_size=256", "+rl_config.clip_higher_enable=true", "+rl_config.clip_ratio_low=0.2",
        "+rl_config.clip_ratio_high=0.28", "+rl_config.token_level_loss=true", "rl_config.init_kl_coef=0.0",
        "generate_config.sampling_config.max_tokens=32", "rl_config.n_samples_per_prompt=4",
        "megatron_training.global_batch_size=8", "rl_config.mini_batch_size=8", "megatron_training.train_iters=2"])
    hist = run_rl(cfg, "dapo")
    if rank == 0:
        assert len(hist) == 2 and all("actor/pg_loss" in m and m["timing/rollout"] > 0 for m in hist)
        assert abs(hist[0]["actor/ppo_kl"]) < 1e-4        # first update: the policy has not moved yet


def test_launch_dapo_long_context_recipe_shape():
    """The long-context DAPO recipes' layout scaled down to 8 ranks: training TP2 x PP2 x CP2 (ring) with sequence
    parallelism, packed sequences and token-budget micro-batches, rollout TP1 x DP8."""
    run_distributed(_launch_dapo_long_context_worker, 8, timeout=280)


def test_launch_grpo_large_expert_recipe_shape():
    """The 235B recipe's structure scaled down to 8 ranks: QK-norm attention, 2 real layers in 4 slots (two empty
    slots) over PP2, training TP2 with the experts spread over TP x EP2, rollout TP4 (TP grows) x EP2."""
    run_distributed(_launch_misc_worker, 8, [
        "actor_config.tensor_model_parallel_size=2", "actor_config.pipeline_model_parallel_size=2",
        "actor_config.expert_model_parallel_size=2", "+actor_config.moe_tp_extend_ep=true",
        "+actor_config.sequence_parallel=true", "+actor_config.no_pad_to_seq_lengths=true",
        "generate_config.infer_tensor_parallel_size=4", "generate_config.infer_expert_parallel_size=2",
        "+model.tiny_qwen2.num_experts=8", "+model.tiny_qwen2.moe_router_topk=2",
        "+model.tiny_qwen2.moe_ffn_hidden_size=32", "+model.tiny_qwen2.norm_topk_prob=true",
        "+model.tiny_qwen2.qk_layernorm=true", "+model.tiny_qwen2.add_qkv_bias=false",
        "+model.tiny_qwen2.num_attention_heads=8", "+model.tiny_qwen2.num_query_groups=4",
        "+actor_config.num_layers=4", "+actor_config.noop_layers='1,3'",
        "generate_config.sampling_config.max_tokens=16", "megatron_training.global_batch_size=8",
        "rl_config.mini_batch_size=8"], "actor/grad_norm", timeout=280)


def _launch_ppo_recipe_worker(rank, world):
    from mindspeed_rl_b200.config import compose
    from mindspeed_rl_b200.runtime.launch import run_rl
    cfg = compose("grpo_tiny_cpu", None, [
        f"rl_config.actor_resource.num_gpus={world}", "megatron_training.stage=ray_ppo", "rl_config.adv_estimator=gae",
        "+critic_config.model=tiny_qwen2", "+critic_config.micro_batch_size=4", "+critic_config.lr=1e-5",
        f"+rl_config.critic_resource.num_gpus={world}", "actor_config.tensor_model_parallel_size=4",
        "+critic_config.tensor_model_parallel_size=4", "+actor_config.sequence_parallel=true",
        "+critic_config.sequence_parallel=true", "generate_config.infer_tensor_parallel_size=2",
        "+actor_config.swap_optimizer=true", "+critic_config.swap_optimizer=true",
        "+model.tiny_qwen2.num_query_groups=4", "+generate_config.offload_train_optimizer=true",
        "+generate_config.offload_train_grad=true", "+generate_config.offload_train_param=true",
        "megatron_training.global_batch_size=4", "rl_config.mini_batch_size=4", "rl_config.n_samples_per_prompt=2",
        "generate_config.sampling_config.max_tokens=8", "megatron_training.train_iters=2"])
    hist = run_rl(cfg, "ppo")
    if rank == 0:
        assert len(hist) == 2
        assert all(m["critic/vf_loss"] >= 0 and m["actor/grad_norm"] > 0 and m["timing/update_critic"] > 0 for m in hist)


def test_launch_ppo_recipe_shape():
    """The PPO recipe's layout scaled down to 4 ranks: actor, reference and critic co-located, training TP4 with
    sequence parallelism and host-resident optimizer state, every offload switch on, rollout TP2 x DP2."""
    run_distributed(_launch_ppo_recipe_worker, 4, timeout=280)


def test_launch_grpo_dense_recipe_shape_with_uneven_stages():
    """The dense recipes' layout scaled down to 4 ranks: training TP2 x PP2 with sequence parallelism, QK-norm
    attention, 4 layers dealt 1 + 3 to the stages (``num_layer_list``), rollout TP1 x DP4."""
    run_distributed(_launch_misc_worker, 4, [
        "actor_config.tensor_model_parallel_size=2", "actor_config.pipeline_model_parallel_size=2",
        "generate_config.infer_tensor_parallel_size=1", "+actor_config.no_pad_to_seq_lengths=true",
        "+actor_config.sequence_parallel=true", "+actor_config.num_layers=4", "+actor_config.num_layer_list='1,3'",
        "+model.tiny_qwen2.qk_layernorm=true", "generate_config.sampling_config.max_tokens=32"],
        "actor/grad_norm", timeout=280)


def _launch_ckpt_worker(rank, world, save, load, iters):
    from mindspeed_rl_b200.config import compose
    from mindspeed_rl_b200.runtime.launch import run_rl
    cfg = compose("grpo_tiny_cpu", None, [
        f"rl_config.actor_resource.num_gpus={world}", "actor_config.tensor_model_parallel_size=2",
        "actor_config.pipeline_model_parallel_size=2", "generate_config.infer_tensor_parallel_size=1",
        "+actor_config.no_pad_to_seq_lengths=true", "+actor_config.sequence_parallel=true",
        "megatron_training.global_batch_size=4", "rl_config.mini_batch_size=4", "rl_config.n_samples_per_prompt=2",
        "generate_config.sampling_config.max_tokens=8", f"megatron_training.train_iters={iters}",
        f"actor_config.save={save}", "megatron_training.save_interval=1"] + ([f"actor_config.load={load}"] if load else []))
    hist = run_rl(cfg, "grpo")
    if rank == 0:
        assert len(hist) == (iters if not load else iters - 2)


def test_checkpoint_of_a_tp_pp_run_resumes_and_converts(tmp_path):
    """A TP2 x PP2 run writes one directory per (TP, PP) rank; a second run resumes from it at the saved
    iteration; the command-line converter turns the shards into Hugging Face tensors and back bit for bit."""
    import importlib
    import sys
    from mindspeed_rl_b200.checkpoint import convert as C
    from mindspeed_rl_b200.config import MegatronConfig
    from mindspeed_rl_b200.config.loader import load_model_catalogue
    save = str(tmp_path / "ckpt")
    run_distributed(_launch_ckpt_worker, 4, save, None, 2, timeout=240)
    it = tmp_path / "ckpt" / "iter_0000002"
    assert sorted(p.name for p in it.iterdir()) == ["mp_rank_00_000", "mp_rank_00_001", "mp_rank_01_000", "mp_rank_01_001"]
    run_distributed(_launch_ckpt_worker, 4, save, save, 3, timeout=240)
    assert (tmp_path / "ckpt" / "latest_checkpointed_iteration.txt").read_text().strip() == "3"
    root = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
    if root not in sys.path:
        sys.path.insert(0, root)
    cli = importlib.import_module("cli.convert_ckpt")
    cli.main(["mcore2hf", "--model", "tiny_qwen2", "--load", save, "--save", str(tmp_path / "hf"), "--tp", "2", "--pp", "2"])
    hf = C.load_hf_state(str(tmp_path / "hf"))
    assert hf["model.embed_tokens.weight"].shape == (1024, 256) and hf["model.layers.1.mlp.gate_proj.weight"].shape == (688, 256)
    cfg = MegatronConfig({"model": "tiny_qwen2"}, load_model_catalogue(["tiny_qwen2"]))
    again, orig = C.hf_to_mcore(hf, cfg, 2, 2), C.read_mcore(save, 2, 2)
    assert sorted(orig) == [(0, 0, 0), (0, 1, 0), (1, 0, 0), (1, 1, 0)]
    for key in orig:
        for name, value in orig[key].items():
            assert torch.equal(again[key][name], value), (key, name)


def _moe_tp_step_worker(rank, world, extend):
    """One optimizer step of an expert model under TP2 with sequence parallelism (experts replicated over the TP
    ranks, or spread over them) equals the step of the single-rank model: the gradient sync adds up the partial
    gradients of routers, norms and replicated experts, and the global gradient norm counts every parameter once."""
    from mindspeed_rl_b200.models.gpt import GPTModel, PackedMeta
    from mindspeed_rl_b200.models.transformer_config import TransformerConfig
    from mindspeed_rl_b200.optim.distributed_optimizer import DistributedOptimizer
    from mindspeed_rl_b200.parallel.ddp import DistributedDataParallel, expert_replica_groups
    from mindspeed_rl_b200.parallel.state import initialize_model_parallel, set_parallel_state
    from mindspeed_rl_b200.parallel.tp_comm import TPComm
    kw = dict(num_layers=2, hidden_size=32, ffn_hidden_size=64, num_attention_heads=4, num_query_groups=2,
              vocab_size=64, add_qkv_bias=True, params_dtype=torch.float32, max_position_embeddings=128,
              num_experts=4, moe_router_topk=2, moe_ffn_hidden_size=16, n_shared_experts=1, moe_aux_loss_coeff=0.0,
              norm_topk_prob=True)
    set_parallel_state(None)
    initialize_model_parallel(world_size=1, rank=0)
    full = DistributedDataParallel(GPTModel(TransformerConfig(**kw), device="cpu", seed=5))
    full_opt = DistributedOptimizer(full.buffers, lr=1e-2, clip_grad=0.5, weight_decay=0.0)
    set_parallel_state(None)
    ps = initialize_model_parallel(tensor_model_parallel_size=world, moe_tp_extend_ep=extend)
    cfg = TransformerConfig(tensor_model_parallel_size=world, sequence_parallel=True, **kw)
    comm = TPComm(ps.group("tp"), True, world_size=world, rank=rank)
    core = GPTModel(cfg, comm, device="cpu")
    ep, er = ps.size("ep"), ps.rank_in("ep")
    h, f, e = 32, 16, 4
    per = e // ep

    def shard(state):
        out = _shard_state(state, cfg, world, rank)
        for k, v in state.items():
            if k.endswith("experts.weight1"):
                out[k] = v.view(h, e, 2 * f)[:, er * per:(er + 1) * per].reshape(h, -1).contiguous()
            elif k.endswith("experts.weight2"):
                out[k] = v.view(e, f, h)[er * per:(er + 1) * per].reshape(-1, h).contiguous()
        return out

    core.load_state_dict(shard({k: v.clone() for k, v in full.module.state_dict().items()}))
    model = DistributedDataParallel(core, ps.group("dp_cp"), 1, **expert_replica_groups(ps, cfg))
    model.attach_tensor_parallel(ps.group("tp"), world, True)
    opt = DistributedOptimizer(model.buffers, lr=1e-2, clip_grad=0.5, weight_decay=0.0, dp_group=ps.group("dp_cp"),
                               dp_rank=0, model_parallel_group=ps.group("mp"), tp_rank=rank)
    meta = PackedMeta.from_lengths([6, 10], "cpu", align=world)
    t = int(meta.cu_seqlens[-1])
    g = torch.Generator().manual_seed(1)
    ids, labels, w = torch.randint(0, 64, (t,), generator=g), torch.randint(0, 64, (t,), generator=g), torch.randn(t, generator=g)
    (full.module.forward_logprob(ids, labels, meta, 0.9, False)[0] * w).sum().backward()
    core.embed = lambda x, _m=core: _seq_shard(_orig_embed(_m, x), world, rank)
    (core.forward_logprob(ids, labels, meta, 0.9, False)[0] * w).sum().backward()
    for p in list(full.module.parameters()) + list(core.parameters()):
        if p.grad is not None:
            p.main_grad.add_(p.grad)
    model.finish_grad_sync(to_shards=True)
    _, norm, _ = opt.step()
    _, full_norm, _ = full_opt.step()
    assert torch.allclose(norm, full_norm, rtol=2e-4), (float(norm), float(full_norm))
    want = shard(full.module.state_dict())
    for k, v in core.state_dict().items():
        assert torch.allclose(v, want[k], atol=5e-5), (k, float((v - want[k]).abs().max()))


def test_expert_layers_under_tensor_parallelism_take_the_single_rank_step():
    run_distributed(_moe_tp_step_worker, 2, False, timeout=240)
    run_distributed(_moe_tp_step_worker, 2, True, timeout=240)


def _launch_dapo_benchmark_shape_worker(rank, world):
    from mindspeed_rl_b200.config import compose
    from mindspeed_rl_b200.runtime.launch import run_rl
    cfg = compose("grpo_tiny_cpu", None, [
        f"rl_config.actor_resource.num_gpus={world}", "megatron_training.stage=ray_dapo",
        "actor_config.tensor_model_parallel_size=4", "actor_config.context_parallel_size=2",
        "actor_config.context_parallel_algo=megatron_cp_algo", "+actor_config.sequence_parallel=true",
        "generate_config.infer_tensor_parallel_size=1", "+model.tiny_qwen2.num_query_groups=4",
        "+model.tiny_qwen2.qk_layernorm=true", "+model.tiny_qwen2.add_qkv_bias=false",
        "rl_config.partial_rollout_max_split=2", "+rl_config.filter_groups_enable=true",
        "+rl_config.filter_groups_metric=contains_token_7", "+rl_config.filter_groups_max_batches=60",
        "+rl_config.filter_groups_train_batch_size=4", "+rl_config.clip_higher_enable=true",
        "+rl_config.clip_ratio_low=0.2", "+rl_config.clip_ratio_high=0.28", "+rl_config.token_level_loss=true",
        "rl_config.init_kl_coef=0.0", "generate_config.sampling_config.max_tokens=32",
        "rl_config.n_samples_per_prompt=4", "megatron_training.global_batch_size=8", "rl_config.mini_batch_size=4",
        "megatron_training.train_iters=2"])
    hist = run_rl(cfg, "dapo")
    if rank == 0:
        assert len(hist) == 2
        assert all(m["train/num_gen_batches"] >= 1 and -1.0 < m["dapo/score/mean"] < 1.0 and m["actor/grad_norm"] > 0
                   for m in hist)


def test_launch_dapo_benchmark_configuration_shape():
    """The DAPO benchmark configuration's structure scaled down to 8 ranks: QK-norm attention, training TP4 x CP2
    (ring) with sequence parallelism, rollout TP1 x DP8, clip-higher, dynamic sampling and partial rollout."""
    run_distributed(_launch_dapo_benchmark_shape_worker, 8, timeout=280)


def test_launch_grpo_with_the_sharded_store_and_the_side_channel():
    """The sharded experience store (``data_strategy: tq``) with the ZeroMQ fan-out inside a TP2 replica."""
    run_distributed(_launch_misc_worker, 2, [
        "+rl_config.data_strategy=tq", "+rl_config.zmq_communication=true",
        "actor_config.tensor_model_parallel_size=2", "generate_config.infer_tensor_parallel_size=2",
        "generate_config.sampling_config.max_tokens=32"], "actor/grad_norm", timeout=240)
