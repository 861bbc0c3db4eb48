"""Multi-GPU cases run under ``torchrun`` by ``test_gpu_multi.py`` (one process per GPU, NCCL).

Usage: ``torchrun --nproc-per-node N tests/multi_gpu_cases.py <case>``.  Every case prints
``CASE <name> OK`` on rank 0 when all ranks agree; any mismatch raises.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _init():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl")
    return rank, world


def case_collectives(rank, world):
    from mindspeed_rl_b200.parallel.symm import SymmetricArena

    arena = SymmetricArena(256 << 20)
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    n = 8 * world * 4099 * 8
    # all-gather (in place into the tensor that holds the source slice)
    full = arena.alloc(n, torch.bfloat16)
    per = n // world
    full[rank * per:(rank + 1) * per].copy_(torch.randn(per, device="cuda", generator=g))
    want = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    dist.all_gather_into_tensor(want, full[rank * per:(rank + 1) * per].clone())
    arena.all_gather_inplace(full)
    arena.check()
    assert torch.equal(full, want), "in-place all_gather mismatch"
    stage = arena.alloc(per, torch.bfloat16)             # same offset on every rank
    stage.copy_(full[rank * per:(rank + 1) * per])
    out = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    arena.all_gather(stage, out)
    arena.check()
    assert torch.equal(out, want), "all_gather mismatch"
    # reduce-scatter bf16 -> own slice in place + fp32 copy
    grads = arena.alloc(n, torch.bfloat16)
    grads.copy_(torch.randn(n, device="cuda", generator=g))
    ref = grads.float().clone()
    dist.all_reduce(ref)
    ref = ref[rank * per:(rank + 1) * per] / world
    out32 = torch.empty(per, dtype=torch.float32, device="cuda")
    arena.reduce_scatter(grads, grads[rank * per:(rank + 1) * per], out_f32=out32, scale=1.0 / world)
    arena.check()
    assert torch.allclose(out32, ref, atol=1e-5, rtol=1e-5), "reduce_scatter fp32 output mismatch"
    assert torch.allclose(grads[rank * per:(rank + 1) * per].float(), ref, atol=2e-2, rtol=2e-2)
    # fp32 reduce-scatter
    g32 = arena.alloc(n, torch.float32)
    g32.copy_(torch.randn(n, device="cuda", generator=g))
    ref = g32.clone()
    dist.all_reduce(ref)
    out = torch.empty(per, dtype=torch.float32, device="cuda")
    arena.reduce_scatter(g32, out)
    arena.check()
    assert torch.allclose(out, ref[rank * per:(rank + 1) * per], atol=1e-5, rtol=1e-5)
    # sub-team barrier / gather (pairs) when there are at least 4 ranks
    if world >= 4:
        pair = [rank - rank % 2, rank - rank % 2 + 1]
        src = arena.alloc(1024, torch.float32)
        src.fill_(float(rank))
        dst = torch.empty(2048, dtype=torch.float32, device="cuda")
        arena.all_gather(src, dst, ranks=pair)
        arena.check()
        assert dst[:1024].eq(pair[0]).all() and dst[1024:].eq(pair[1]).all()
    arena.close()


def case_peer_all_reduce(rank, world):
    """The small-message all-reduce of the decode step: against the library collective (bit-identical
    results on all ranks), over many consecutive calls with changing sizes (parity double-buffering),
    in place, replayed from a CUDA graph, and on sub-teams of two when there are four ranks or more."""
    from mindspeed_rl_b200.parallel.symm import SymmetricArena

    arena = SymmetricArena(256 << 20)
    ar = arena.make_all_reduce(1024 * 3584 * 2)
    g = torch.Generator(device="cuda").manual_seed(7 + rank)
    for call, tokens in enumerate([256, 1, 8, 512, 1024, 3, 256, 256, 64, 1000]):
        x = torch.randn(tokens, 3584, device="cuda", generator=g).bfloat16()
        want = x.float()
        dist.all_reduce(want)
        got = ar.all_reduce(x.clone())
        arena.check()
        assert torch.allclose(got.float(), want, atol=2e-2 * world, rtol=2e-2), (call, (got.float() - want).abs().max())
        every = [torch.empty_like(got) for _ in range(world)]
        dist.all_gather(every, got)
        assert all(torch.equal(every[0], e) for e in every), f"call {call}: ranks disagree bit-wise"
    assert not ar.fits(torch.empty(2048, 3584, device="cuda", dtype=torch.bfloat16))
    # CUDA-graph replay: the launch reads its sequence number from device memory
    static = torch.zeros(256, 3584, device="cuda", dtype=torch.bfloat16)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        ar.all_reduce(static)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ar.all_reduce(static)
        ar.all_reduce(static)
    for it in range(5):
        static.fill_(float(rank + it))
        graph.replay()
        arena.check()
        s1 = sum(r + it for r in range(world))
        assert torch.all(static.float() == float(s1 * world)), (it, static[0, 0])
    if world >= 4:
        pair = [rank - rank % 2, rank - rank % 2 + 1]
        sub = arena.make_all_reduce(64 * 1024, pair)
        y = torch.full((8, 1024), float(rank), device="cuda", dtype=torch.bfloat16)
        sub.all_reduce(y)
        arena.check()
        assert torch.all(y.float() == float(pair[0] + pair[1]))

    arena.check()
    arena.close()


def case_reshard(rank, world):
    """Train TP=world -> rollout TP=1 and TP=world/2 through the copy-plan kernel vs the torch executor."""
    from mindspeed_rl_b200.models.gpt import GPTModel
    from mindspeed_rl_b200.models.transformer_config import TransformerConfig
    from mindspeed_rl_b200.parallel.ddp import DistributedDataParallel
    from mindspeed_rl_b200.parallel.state import initialize_model_parallel
    from mindspeed_rl_b200.parallel.symm import init_arena
    from mindspeed_rl_b200.parallel.tp_comm import TPComm
    from mindspeed_rl_b200.reshard.planner import Resharder

    ps = initialize_model_parallel(world)
    cfg = TransformerConfig(num_layers=3, hidden_size=256, ffn_hidden_size=512, num_attention_heads=8,
                            num_query_groups=4, vocab_size=1024, kv_channels=32, add_qkv_bias=True,
                            tensor_model_parallel_size=world)
    comm = TPComm(ps.group("tp"), False, world_size=world, rank=rank)
    init_arena(128 << 20)
    core = GPTModel(cfg, comm, device="cuda", seed=5)
    ddp = DistributedDataParallel(core, None, 1)
    assert ddp.buffers[0].arena is not None

    class _Engine:
        def __init__(self, *a):
            pass

    for infer_tp in sorted({1, max(world // 2, 1)}):
        rs = Resharder(cfg, ddp, ps, infer_tp, "cuda", lambda c, comm_: _Engine(), arena=ddp.buffers[0].arena)
        w = rs.reshard(core)
        assert rs._plan_dev is not None, "the peer-memory path was not taken"
        got = rs.buffer.clone()
        rs.arena.check()
        rs.arena = None                      # same plan through the gathered (NCCL) fallback
        rs._plan = None
        rs.buffer = torch.zeros_like(got)
        rs.reshard(core)
        assert torch.equal(got, rs.buffer), f"copy-plan kernel differs from the oracle (infer_tp={infer_tp})"
        assert w.layers[0].o_w.shape == (cfg.hidden_size, cfg.num_attention_heads * 32 // infer_tp)


def case_fused_tp(rank, world):
    """all-gather->GEMM and GEMM->reduce-scatter tcgen05 kernels against NCCL + matmul."""
    from mindspeed_rl_b200.ops.gemm import check_status
    from mindspeed_rl_b200.parallel.fused_tp import FusedTP
    from mindspeed_rl_b200.parallel.symm import SymmetricArena

    small = os.environ.get("MSRL_TEST_SMALL", "0") == "1"
    ml, hidden, n_col, k_row = (256, 512, 768, 256) if small else (2048, 3584, 4608 // world * 2, 18944 // world // 8 * 8)
    arena = SymmetricArena((6 * ml * max(hidden, n_col) * 2 * (world + 1)) + (64 << 20))
    f = FusedTP(arena, list(range(world)), ml, hidden, hidden)
    g = torch.Generator(device="cuda").manual_seed(7 + rank)
    rnd = lambda *s: (torch.randn(*s, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    ml_max = ml
    # many consecutive calls with changing token counts: parity buffers, counter re-arming, both the
    # CTA-pair kernels (shards in multiples of 256 rows) and the single-CTA ones (multiples of 128)
    shapes = [ml_max, ml_max, ml_max // 4, ml_max // 4 + 128, ml_max // 2 + 256, ml_max, ml_max // 8, ml_max]
    for it, ml in enumerate(shapes):
        x, w = rnd(ml, hidden), rnd(n_col, hidden)
        y, xg = f.ag_gemm(x, w)
        want_x = torch.empty(world * ml, hidden, dtype=torch.bfloat16, device="cuda")
        dist.all_gather_into_tensor(want_x, x)
        check_status(torch.device("cuda", torch.cuda.current_device()),"ag_gemm")
        assert torch.equal(xg, want_x), f"gathered activations differ (call {it})"
        ref = torch.matmul(want_x.float(), w.float().t())
        err = (y.float() - ref).abs().max().item()
        assert err <= 2e-2 * ref.abs().max().item() + 1e-3, f"ag_gemm error {err} (call {it})"
        a, w2 = rnd(world * ml, k_row), rnd(hidden, k_row)
        out = f.gemm_rs(a, w2)
        part = torch.matmul(a, w2.t())
        want = torch.empty(ml, hidden, dtype=torch.bfloat16, device="cuda")
        dist.reduce_scatter_tensor(want, part)
        check_status(torch.device("cuda", torch.cuda.current_device()),"gemm_rs")
        ref = want.float()
        err = (out.float() - ref).abs().max().item()
        assert err <= 3e-2 * ref.abs().max().item() + 1e-3, f"gemm_rs error {err} (call {it})"

    arena.check()
    arena.close()


def case_tp_model(rank, world):
    """Sequence-parallel TP model: forward + backward with the fused linears attached equals the
    NCCL + matmul path on the same weights (bf16 tolerances)."""
    from mindspeed_rl_b200.models.gpt import GPTModel, PackedMeta
    from mindspeed_rl_b200.models.transformer_config import TransformerConfig
    from mindspeed_rl_b200.ops.gemm import check_status
    from mindspeed_rl_b200.parallel.ddp import DistributedDataParallel
    from mindspeed_rl_b200.parallel.fused_tp import FusedTP
    from mindspeed_rl_b200.parallel.state import initialize_model_parallel
    from mindspeed_rl_b200.parallel.symm import init_arena
    from mindspeed_rl_b200.parallel.tp_comm import TPComm

    ps = initialize_model_parallel(world)
    cfg = TransformerConfig(num_layers=2, hidden_size=512, ffn_hidden_size=1024, num_attention_heads=8,
                            num_query_groups=4, vocab_size=2048, kv_channels=64, add_qkv_bias=True,
                            tensor_model_parallel_size=world, sequence_parallel=True)
    comm = TPComm(ps.group("tp"), True, world_size=world, rank=rank)
    arena = init_arena(256 << 20)
    model = DistributedDataParallel(GPTModel(cfg, comm, device="cuda", seed=11), None, 1)
    core = model.module
    lens = [128 * world, 128 * world]
    meta = PackedMeta.from_lengths(lens, "cuda", align=world)
    t = int(meta.cu_seqlens[-1])
    g = torch.Generator(device="cuda").manual_seed(1)
    ids = torch.randint(0, 2048, (t,), device="cuda", generator=g)
    labels = torch.randint(0, 2048, (t,), device="cuda", generator=g)
    wts = torch.randn(t, device="cuda", generator=g)

    def run():
        model.zero_grad_buffer()
        lp, _ = core.forward_logprob(ids, labels, meta, 1.0, False)
        (lp * wts).sum().backward()
        return lp.detach().clone(), [b.grad_data.float().clone() for b in model.buffers]

    lp_ref, g_ref = run()
    comm.fused = FusedTP(arena, list(range(world)), t // world, cfg.hidden_size, cfg.hidden_size)
    calls = comm.fused._ag_calls
    lp, g_f = run()
    check_status(torch.device("cuda", torch.cuda.current_device()), "fused tp model")
    arena.check()
    assert comm.fused._ag_calls > calls and comm.fused._rs_calls > 0, "the fused kernels were not used"
    assert (lp - lp_ref).abs().max().item() < 5e-2, (lp - lp_ref).abs().max().item()
    for a, b in zip(g_f, g_ref):
        denom = b.abs().max().item() + 1e-6
        assert (a - b).abs().max().item() / denom < 5e-2, ((a - b).abs().max().item(), denom)


def case_grpo_reshard(rank, world):
    """One GRPO iteration with train TP=2 and rollout TP=1 (resharding through peer memory)."""
    from mindspeed_rl_b200.config import compose, parse_training_config  # noqa: F401
    from mindspeed_rl_b200.runtime.launch import run_rl

    cfg = compose("grpo_tiny_cpu", None, [
        "actor_config.tensor_model_parallel_size=2", "generate_config.infer_tensor_parallel_size=1",
        "rl_config.actor_resource.num_gpus=%d" % world])
    hist = run_rl(cfg, "grpo")
    if rank == 0:
        assert len(hist) == 2, hist


def case_moe_ep_p2p(rank, world):
    """Expert parallelism with tokens written straight into the destination ranks' expert slabs
    (peer-mapped memory) and outputs pulled back by the source ranks."""
    case_moe_ep(rank, world, p2p_rows=4096)


def case_moe_ep(rank, world, p2p_rows=0):
    """Expert parallelism on GPUs (token exchange over NCCL, local experts on the plan + grouped tcgen05
    GEMM kernels) against the same model with all experts on one rank."""
    from mindspeed_rl_b200.models.gpt import GPTModel, PackedMeta
    from mindspeed_rl_b200.models.transformer_config import TransformerConfig
    from mindspeed_rl_b200.ops.gemm import check_status
    from mindspeed_rl_b200.parallel.state import initialize_model_parallel, set_parallel_state
    e, h, f = 8, 256, 128
    kw = dict(num_layers=1, hidden_size=h, ffn_hidden_size=512, num_attention_heads=4, num_query_groups=2,
              vocab_size=512, kv_channels=64, max_position_embeddings=1024, num_experts=e, moe_router_topk=2,
              moe_ffn_hidden_size=f, norm_topk_prob=True, moe_aux_loss_coeff=0.0)
    set_parallel_state(None)
    full = GPTModel(TransformerConfig(**kw), device="cuda", seed=3)
    initialize_model_parallel(expert_model_parallel_size=world)
    arena = None
    if p2p_rows:
        from mindspeed_rl_b200.parallel.symm import init_arena
        arena = init_arena(64 << 20)
    model = GPTModel(TransformerConfig(expert_model_parallel_size=world, moe_p2p_dispatch_rows=p2p_rows, **kw),
                     device="cuda", seed=3)
    sd = full.state_dict()
    per = e // world
    for k in list(sd):
        if k.endswith("experts.weight1"):
            sd[k] = sd[k].view(h, e, 2 * f)[:, rank * per:(rank + 1) * per].reshape(h, -1).contiguous()
        if k.endswith("experts.weight2"):
            sd[k] = sd[k].view(e, f, h)[rank * per:(rank + 1) * per].reshape(-1, h).contiguous()
    model.load_state_dict(sd)
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    lens = [300, 212]
    meta = PackedMeta.from_lengths(lens, "cuda")
    t = sum(lens)
    ids = torch.randint(0, 512, (t,), device="cuda", generator=g)
    labels = torch.randint(0, 512, (t,), device="cuda", generator=g)
    ref, _ = full.forward_logprob(ids, labels, meta)
    ref.sum().backward()
    lp, _ = model.forward_logprob(ids, labels, meta)
    lp.sum().backward()
    check_status(torch.device("cuda", torch.cuda.current_device()), "moe ep")
    # the rollout view of the layer (forward only, same dispatcher) agrees with the training forward
    layer = model.decoder.layers[0]
    xs = torch.randn(257 + 64 * rank, h, device="cuda", generator=g).bfloat16()
    with torch.no_grad():
        y_train, _ = layer.mlp.forward_tokens(xs, layer.comm, False)
        y_roll = layer.mlp.rollout_view().forward(xs, None)
    assert (y_train.float() - y_roll.float()).abs().max().item() <= 2e-2 * y_train.float().abs().max().item() + 1e-3
    if p2p_rows:
        from mindspeed_rl_b200.parallel import moe_dispatch
        arena.check()
        used = [d for d in moe_dispatch._dispatchers.values() if d is not None]
        assert used and used[0].calls >= 2, "the peer-memory dispatcher was not used"
    assert (lp - ref).abs().max().item() < 5e-2, (lp - ref).abs().max().item()
    gw = model.decoder.layers[0].mlp.experts.weight2.grad.float().view(per, f, h)
    fw = full.decoder.layers[0].mlp.experts.weight2.grad.float().view(e, f, h).clone()
    dist.all_reduce(fw)
    ref_g = fw[rank * per:(rank + 1) * per]
    assert (gw - ref_g).abs().max().item() / (ref_g.abs().max().item() + 1e-6) < 5e-2


def case_cp_ring(rank, world):
    """Ring attention over the context-parallel group (K/V rotation over NCCL p2p, tcgen05 block
    kernels with separate q / kv) against the same model on one GPU."""
    os.environ["MSRL_CP_RING"] = "1"
    from mindspeed_rl_b200.models.gpt import GPTModel, PackedMeta
    from mindspeed_rl_b200.models.transformer_config import TransformerConfig
    from mindspeed_rl_b200.ops.gemm import check_status
    from mindspeed_rl_b200.parallel.context_parallel import ContextParallel
    from mindspeed_rl_b200.parallel.state import initialize_model_parallel
    ps = initialize_model_parallel(context_parallel_size=world)
    cfg = TransformerConfig(num_layers=2, hidden_size=512, ffn_hidden_size=1024, num_attention_heads=4,
                            num_query_groups=2, vocab_size=1024, kv_channels=128, add_qkv_bias=True,
                            max_position_embeddings=4096)
    full = GPTModel(cfg, device="cuda", seed=5)
    model = GPTModel(cfg, device="cuda", seed=5)
    meta = PackedMeta.from_lengths([600, 1300, 404], "cuda", align=2 * world)
    t = int(meta.cu_seqlens[-1])
    g = torch.Generator(device="cuda").manual_seed(1)
    ids = torch.randint(0, 1024, (t,), device="cuda", generator=g)
    labels = torch.randint(0, 1024, (t,), device="cuda", generator=g)
    w = torch.randn(t, device="cuda", generator=g)
    ref_lp, _ = full.forward_logprob(ids, labels, meta, 1.0, False)
    (ref_lp * w).sum().backward()
    cp = ContextParallel(ps.group("cp"), world, rank, "megatron_cp_algo", meta.cu_seqlens.to(torch.int64).cpu(), "cuda")
    assert cp.use_ring(model.decoder.layers[0].self_attention.layout)
    m_local = PackedMeta(cp.cu_local, cp.max_local, cp.take_local(meta.positions), cp=cp)
    lp_l, _ = model.forward_logprob(cp.take_local(ids), cp.take_local(labels), m_local, 1.0, False)
    lp = cp.gather_tokens(lp_l)
    assert (lp - ref_lp).abs().max().item() < 5e-2, (lp - ref_lp).abs().max().item()
    (lp * w).sum().backward()
    check_status(torch.device("cuda", torch.cuda.current_device()), "cp ring")
    for (n, p), q in zip(model.named_parameters(), full.parameters()):
        gr = p.grad.float().clone()
        dist.all_reduce(gr)
        ref = q.grad.float()
        assert (gr / world - ref).abs().max().item() <= 5e-2 * ref.abs().max().item() + 1e-3, \
            (n, (gr / world - ref).abs().max().item(), ref.abs().max().item())


def case_buffer_release(rank, world):
    """Flat buffers with peer-mapped segments of their own: the pull-kernel reduce-scatter / all-gather work
    on them, releasing them gives the memory back to the device, and after restoring them the parameters are
    intact and the collectives work again."""
    from mindspeed_rl_b200.parallel.ddp import DistributedDataParallel
    from mindspeed_rl_b200.parallel.symm import init_arena
    from mindspeed_rl_b200.reshard.sharding_manager import GradBufferOffloader, ParamOffloader

    init_arena(32 << 20)
    torch.manual_seed(5)
    net = torch.nn.Sequential(torch.nn.Linear(4096, 4096, bias=False), torch.nn.Linear(4096, 2048, bias=False))
    net = net.to("cuda", torch.bfloat16)
    ddp = DistributedDataParallel(net, dist.group.WORLD, world, releasable_params=True, releasable_grads=True)
    buf = ddp.buffers[0]
    assert buf._own == {"param": True, "grad": True} and buf.param_arena is not buf.grad_arena
    want_params = buf.param_data.clone()

    def reduce_and_check(seed):
        g = torch.Generator(device="cuda").manual_seed(seed + rank)
        buf.grad_data.copy_(torch.randn(buf.numel, device="cuda", generator=g))
        ref = buf.grad_data.float().clone()
        dist.all_reduce(ref)
        ddp.finish_grad_sync(to_shards=True)
        buf.grad_arena.check()
        s, e = buf.shard_range()
        assert torch.allclose(buf.grad_data[s:e].float(), ref[s:e] / world, atol=2e-2, rtol=2e-2)

    reduce_and_check(10)
    grads, params = GradBufferOffloader(ddp), ParamOffloader(ddp)
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    grads.release()
    params.offload()
    torch.cuda.synchronize()
    free1 = torch.cuda.mem_get_info()[0]
    assert free1 - free0 >= 2 * buf.numel * 2 - (8 << 20), (free0, free1)      # both 48 MB buffers went back
    assert buf.grad_data.numel() == 0 and buf.param_data.numel() == 0 and net[0].weight.main_grad is None
    params.onload()
    grads.restore()
    assert buf.param_arena is not None and buf.grad_arena is not None
    assert torch.equal(buf.param_data, want_params) and net[0].weight.data_ptr() == buf.param_data.data_ptr()
    reduce_and_check(20)
    # parameter all-gather on the restored segment: every rank rewrites its own shard, all see all shards
    s, e = buf.shard_range()
    buf.param_data[s:e].fill_(float(rank + 1))
    buf.gather_params()
    buf.param_arena.check()
    per = buf.numel // world
    for r in range(world):
        assert torch.all(buf.param_data[r * per:(r + 1) * per].float() == float(r + 1))


def case_overlap(rank, world):
    """Data-parallel training steps with the gradient reduction started from the layers' backward and the
    parameter all-gather pipelined behind the optimizer's chunks, both on peer-mapped buffers, against the
    plain path (library collectives after the backward) on ordinary allocations."""
    from mindspeed_rl_b200.models.gpt import GPTModel, PackedMeta
    from mindspeed_rl_b200.models.transformer_config import TransformerConfig
    from mindspeed_rl_b200.optim.distributed_optimizer import DistributedOptimizer
    from mindspeed_rl_b200.parallel.ddp import DistributedDataParallel
    from mindspeed_rl_b200.parallel.state import initialize_model_parallel
    from mindspeed_rl_b200.parallel.symm import get_arena, init_arena

    ps = initialize_model_parallel()
    cfg = TransformerConfig(num_layers=3, hidden_size=256, ffn_hidden_size=512, num_attention_heads=4,
                            num_query_groups=2, vocab_size=1024, max_position_embeddings=256)

    def train(overlap: bool):
        core = GPTModel(cfg, device="cuda", seed=11)
        ddp = DistributedDataParallel(core, ps.group("dp_cp"), world)
        assert (ddp.buffers[0].grad_arena is not None) == overlap
        if overlap:
            ddp.enable_grad_overlap(bucket_numel=300_000)
            assert len(ddp.buffers[0].bucket_ranges) >= 3
        opt = DistributedOptimizer(ddp.buffers, lr=1e-3, betas=(0.9, 0.95), weight_decay=0.0, clip_grad=1.0,
                                   dp_group=ps.group("dp_cp"), dp_rank=rank, overlap_param_gather=overlap,
                                   gather_chunks=4)
        g = torch.Generator(device="cuda").manual_seed(5 + rank)
        for step in range(3):
            ddp.zero_grad_buffer()
            for micro in range(2):
                meta = PackedMeta.from_lengths([70, 58], "cuda")
                ids = torch.randint(0, 1024, (128,), device="cuda", generator=g)
                labels = torch.randint(0, 1024, (128,), device="cuda", generator=g)
                if micro == 1:
                    ddp.begin_last_microbatch()
                lp, _ = core.forward_logprob(ids, labels, meta, 1.0, False)
                (-lp.mean()).backward()
            ddp.finish_grad_sync(to_shards=True)
            opt.step()
            if get_arena() is not None:
                get_arena().check()
        return torch.cat([p.detach().float().reshape(-1) for p in core.parameters()])

    plain = train(False)                 # no arena yet: ordinary buffers, NCCL collectives
    init_arena(64 << 20)
    fused = train(True)
    every = [torch.empty_like(fused) for _ in range(world)]
    dist.all_gather(every, fused)
    assert all(torch.equal(every[0], e) for e in every), "ranks hold different parameters after the pipelined gather"
    err = (plain - fused).abs().max().item()
    assert err <= 2e-2, err              # bf16 parameters, different summation orders


def case_arena_fallback(rank, world):
    """One rank cannot allocate its arena (it asks for far more than the device has; the allocation
    call returns an error code): every rank gets the same exception, nobody is left waiting in a
    collective, and a normal arena can be created afterwards."""
    from mindspeed_rl_b200.parallel.symm import ArenaUnavailable, get_arena, init_arena
    try:
        init_arena((1 << 45) if rank == world - 1 else (8 << 20))
        raise AssertionError("the oversized arena must not come up")
    except ArenaUnavailable as e:
        assert f"[{world - 1}]" in str(e), str(e)
    assert get_arena() is None
    arena = init_arena(8 << 20)
    x = arena.alloc(1024, torch.float32)
    x.fill_(float(rank + 1))
    arena.barrier()
    arena.check()
    torch.cuda.synchronize()
    assert float(x[0]) == rank + 1


CASES = {"peer_all_reduce": case_peer_all_reduce, "overlap": case_overlap, "buffer_release": case_buffer_release, "arena_fallback": case_arena_fallback, "cp_ring": case_cp_ring, "moe_ep": case_moe_ep, "moe_ep_p2p": case_moe_ep_p2p, "collectives": case_collectives, "reshard": case_reshard, "grpo_reshard": case_grpo_reshard,
         "fused_tp": case_fused_tp, "tp_model": case_tp_model}

if __name__ == "__main__":
    name = sys.argv[1]
    if name == "grpo_reshard":
        CASES[name](int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]))
    else:
        r, w = _init()
        CASES[name](r, w)
        torch.cuda.synchronize()
        dist.barrier()
    if int(os.environ["RANK"]) == 0:
        print(f"CASE {name} OK", flush=True)
    if dist.is_initialized():
        dist.destroy_process_group()
