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
    # timing: device time of the pull kernels against NCCL on the same sizes
    big = arena.alloc(64 << 20, torch.bfloat16)
    bper = big.numel() // world
    tmp = torch.empty_like(big)

    def timed(fn, iters=5):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / iters], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    t_ag = timed(lambda: arena.all_gather_inplace(big))
    t_ag_nccl = timed(lambda: dist.all_gather_into_tensor(tmp, big[rank * bper:(rank + 1) * bper]))
    t_rs = timed(lambda: arena.reduce_scatter(big, big[rank * bper:(rank + 1) * bper], scale=0.5))
    t_rs_nccl = timed(lambda: dist.reduce_scatter_tensor(tmp[rank * bper:(rank + 1) * bper], big))
    arena.check()
    if rank == 0:
        mb = big.numel() * 2 / 1e6
        print(f"TIMING world={world} size={mb:.0f}MB all_gather symm={t_ag:.3f}ms nccl={t_ag_nccl:.3f}ms "
              f"reduce_scatter symm={t_rs:.3f}ms nccl={t_rs_nccl:.3f}ms", flush=True)
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


CASES = {"collectives": case_collectives, "reshard": case_reshard, "grpo_reshard": case_grpo_reshard}

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
