"""Multi-GPU micro-benchmarks: device time (CUDA events, max over ranks) of the peer-memory kernels
against the library collectives they replace.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m mindspeed_rl_b200.ops.microbench_multi [--only collectives,peer_all_reduce,fused_tp,moe_dispatch,tp_layers]

One process per GPU over NCCL.  Rank 0 prints one JSON line per case.  Correctness of the same kernels is
covered by the multi-GPU tests; this module only times them.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def timed(fn, iters: int = 10, warmup: int = 3) -> float:
    """Milliseconds per call: CUDA events around ``iters`` back-to-back calls after warm-up, ranks
    lined up before the first timed call, maximum over ranks."""
    for _ in range(warmup):
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


def report(rank: int, **kw) -> None:
    if rank == 0:
        print(json.dumps({k: (round(v, 4) if isinstance(v, float) else v) for k, v in kw.items()}), flush=True)


def case_collectives(rank: int, world: int) -> None:
    """Pull-kernel all-gather / reduce-scatter of a 128 MB bf16 buffer against NCCL."""
    from ..parallel.symm import SymmetricArena

    arena = SymmetricArena(192 << 20)
    big = arena.alloc(64 << 20, torch.bfloat16)
    per = big.numel() // world
    tmp = torch.empty_like(big)
    t_ag = timed(lambda: arena.all_gather_inplace(big), 5, 2)
    t_ag_nccl = timed(lambda: dist.all_gather_into_tensor(tmp, big[rank * per:(rank + 1) * per]), 5, 2)
    t_rs = timed(lambda: arena.reduce_scatter(big, big[rank * per:(rank + 1) * per], scale=0.5), 5, 2)
    t_rs_nccl = timed(lambda: dist.reduce_scatter_tensor(tmp[rank * per:(rank + 1) * per], big), 5, 2)
    arena.check()
    report(rank, case="collectives", world=world, mbytes=big.numel() * 2 / 1e6, all_gather_symm_ms=t_ag,
           all_gather_nccl_ms=t_ag_nccl, reduce_scatter_symm_ms=t_rs, reduce_scatter_nccl_ms=t_rs_nccl)
    arena.close()


def case_peer_all_reduce(rank: int, world: int) -> None:
    """The decode step's small all-reduce (tokens x 3584 bf16) through peer stores against NCCL."""
    from ..parallel.symm import SymmetricArena

    arena = SymmetricArena(64 << 20)
    ar = arena.make_all_reduce(1024 * 3584 * 2)
    for tokens in (64, 256, 512):
        x = torch.randn(tokens, 3584, device="cuda").bfloat16()
        t_peer = timed(lambda: ar.all_reduce(x), 50, 5)
        t_nccl = timed(lambda: dist.all_reduce(x), 50, 5)
        report(rank, case="peer_all_reduce", world=world, tokens=tokens, mbytes=tokens * 7168 / 1e6,
               peer_us=t_peer * 1e3, nccl_us=t_nccl * 1e3)
    arena.check()
    arena.close()


def case_fused_tp(rank: int, world: int) -> None:
    """all-gather -> GEMM and GEMM -> reduce-scatter as one kernel each (CTA-pair and single-CTA
    variants) against NCCL + library GEMM, on the 7B attention / MLP shapes of one TP rank."""
    from ..ops.gemm import check_status
    from ..parallel.fused_tp import FusedTP
    from ..parallel.symm import SymmetricArena

    ml = int(os.environ.get("MSRL_BENCH_M_LOCAL", "2048"))
    hidden, n_col, k_row = 3584, 4608 // world * 2, 18944 // world // 8 * 8
    arena = SymmetricArena((6 * ml * max(hidden, n_col) * 2 * (world + 1)) + (64 << 20))
    f = FusedTP(arena, list(range(world)), ml, hidden, hidden)
    g = torch.Generator(device="cuda").manual_seed(7 + rank)
    rnd = lambda *s: (torch.randn(*s, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    x, w = rnd(ml, hidden), rnd(n_col, hidden)
    a, w2 = rnd(world * ml, k_row), rnd(hidden, k_row)
    xg = torch.empty(world * ml, hidden, dtype=torch.bfloat16, device="cuda")
    o = torch.empty(ml, hidden, dtype=torch.bfloat16, device="cuda")

    def base_ag():
        dist.all_gather_into_tensor(xg, x)
        return torch.matmul(xg, w.t())

    def base_rs():
        dist.reduce_scatter_tensor(o, torch.matmul(a, w2.t()))

    t = dict(ag_pair=timed(lambda: f.ag_gemm(x, w)), ag_nccl_cublas=timed(base_ag),
             rs_pair=timed(lambda: f.gemm_rs(a, w2)), rs_cublas_nccl=timed(base_rs))
    f.use_pair = False
    t.update(ag_single=timed(lambda: f.ag_gemm(x, w)), rs_single=timed(lambda: f.gemm_rs(a, w2)))
    check_status(torch.device("cuda", torch.cuda.current_device()), "fused timing loop")
    arena.check()
    report(rank, case="fused_tp", world=world, m_local=ml, ag_shape=[world * ml, n_col, hidden],
           rs_shape=[world * ml, hidden, k_row], ag_tflops=2.0 * world * ml * hidden * n_col / t["ag_pair"] / 1e9,
           rs_tflops=2.0 * world * ml * k_row * hidden / t["rs_pair"] / 1e9, **{k + "_ms": v for k, v in t.items()})
    arena.close()


def case_moe_dispatch(rank: int, world: int) -> None:
    """One MoE token round trip between expert-parallel ranks: peer-memory dispatch + combine against
    count exchange + two all-to-all collectives."""
    from ..parallel.moe_dispatch import P2PDispatcher
    from ..parallel.symm import SymmetricArena

    t, k, h, e_local = 8192, 8, 2048, 16
    e = e_local * world
    rows = 2 * t * k + e_local * 128
    arena = SymmetricArena(P2PDispatcher.bytes_needed(world, e_local, h, rows) + (8 << 20))
    disp = P2PDispatcher(arena, list(range(world)), e_local, h, rows, fallback=False)
    g = torch.Generator(device="cuda").manual_seed(rank)
    x = torch.randn(t, h, device="cuda", generator=g).bfloat16()
    idx = torch.stack([torch.randperm(e, device="cuda", generator=g)[:k] for _ in range(256)]).repeat(t // 256, 1)
    w = torch.rand(t, k, device="cuda", generator=g)

    def p2p():
        route = disp.dispatch(x, idx)
        disp.out_slab.copy_(disp.slab)                      # stand-in for the expert MLP
        return disp.combine(route, w)[0]

    def a2a():
        flat = idx.reshape(-1)
        order = torch.argsort(flat, stable=True)
        xp = x[order // k]
        send = torch.bincount(flat, minlength=e).view(world, e_local)
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send)
        send_rows, recv_rows = send.sum(1).tolist(), recv.sum(1).tolist()
        got = torch.empty(sum(recv_rows), h, device="cuda", dtype=x.dtype)
        dist.all_to_all_single(got, xp, recv_rows, send_rows)
        back = torch.empty_like(xp)
        dist.all_to_all_single(back, got, send_rows, recv_rows)
        out = torch.zeros(t, h, device="cuda", dtype=torch.float32)
        out.index_add_(0, order // k, (back * w.reshape(-1)[order].to(x.dtype).unsqueeze(-1)).float())
        return out.to(x.dtype)

    t_p2p, t_a2a = timed(p2p), timed(a2a)
    arena.check()
    report(rank, case="moe_dispatch", world=world, tokens_per_rank=t, topk=k, hidden=h, p2p_ms=t_p2p, nccl_a2a_ms=t_a2a)
    arena.close()


def case_tp_layers(rank: int, world: int) -> None:
    """A few 7B layers + LM head under tensor / sequence parallelism over all ranks: time per forward and
    per forward + backward with the communication-fused linears and with library collectives around plain
    GEMMs (``MSRL_BENCH_KERNEL_TABLE=1`` adds the top kernels by device time from ``torch.profiler``)."""
    from ..models.gpt import GPTModel, PackedMeta
    from ..models.transformer_config import TransformerConfig
    from ..parallel.ddp import DistributedDataParallel
    from ..parallel.fused_tp import FusedTP
    from ..parallel.state import initialize_model_parallel
    from ..parallel.symm import init_arena
    from ..parallel.tp_comm import TPComm

    ps = initialize_model_parallel(world, 1, 1)
    tokens = int(os.environ.get("MSRL_BENCH_TOKENS_PER_RANK", "8192")) * world
    layers = int(os.environ.get("MSRL_BENCH_LAYERS", "4"))
    cfg = TransformerConfig(num_layers=layers, hidden_size=3584, ffn_hidden_size=18944, num_attention_heads=28,
                            num_query_groups=4, vocab_size=152064, add_qkv_bias=True,
                            tensor_model_parallel_size=world, sequence_parallel=world > 1, recompute_granularity=None,
                            recompute_activation_function=True, max_position_embeddings=4096)
    comm = TPComm(ps.group("tp"), True, world_size=world, rank=rank)
    ml = tokens // world
    arena = init_arena(int(2.5e9) + 2 * ml * 3584 * 2 * (1 + world) * 2, device=torch.device("cuda"))
    core = GPTModel(cfg, comm, device="cuda", seed=1)
    DistributedDataParallel(core, None, 1)
    fused = FusedTP(arena, list(range(world)), ml, 3584, 3584) if world > 1 else None
    meta = PackedMeta.from_lengths([2048] * (tokens // 2048), "cuda", align=world)
    ids = torch.randint(0, 150000, (tokens,), device="cuda")
    labels = torch.randint(0, 150000, (tokens,), device="cuda")

    def fwd():
        with torch.no_grad():
            return core.forward_logprob(ids, labels, meta, 1.0, False)[0]

    def fwdbwd():
        core.forward_logprob(ids, labels, meta, 1.0, False)[0].sum().backward()

    out = dict(case="tp_layers", world=world, tokens=tokens, layers=layers)
    for use_fused in ((True, False) if fused is not None else (False,)):
        comm.fused = fused if use_fused else None
        tag = "fused" if use_fused else "library"
        out[f"fwd_{tag}_ms"] = timed(fwd, 3, 2)
        out[f"fwdbwd_{tag}_ms"] = timed(fwdbwd, 3, 2)
        if os.environ.get("MSRL_BENCH_KERNEL_TABLE") == "1":
            from torch.profiler import ProfilerActivity, profile

            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                fwdbwd()
                torch.cuda.synchronize()
            if rank == 0:
                rows = sorted(prof.key_averages(), key=lambda k: -k.device_time_total)[:16]
                total = sum(k.device_time_total for k in prof.key_averages())
                for k in rows:
                    print(f"  [{tag}] {k.device_time_total / 1e3:9.2f} ms {100 * k.device_time_total / total:5.1f}% "
                          f"x{k.count:4d}  {k.key[:90]}", flush=True)
    report(rank, **out)


CASES = {"collectives": case_collectives, "peer_all_reduce": case_peer_all_reduce, "fused_tp": case_fused_tp,
         "moe_dispatch": case_moe_dispatch, "tp_layers": case_tp_layers}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl")
    for name in ([n for n in args.only.split(",") if n] or [n for n in CASES if n != "tp_layers"]):
        CASES[name](rank, world)
        dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
