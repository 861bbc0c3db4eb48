"""Kernel micro-benchmarks: CUDA-event timings and roofline fractions of the hand-written kernels.

    python -m mindspeed_rl_b200.ops.microbench [--only NAME[,NAME..]] [--small] [--iters N]

Each case reports the time per call (median of ``iters`` after warm-up; the L2 is flushed between
timed calls by writing a 256 MiB buffer and then reading another), the achieved bandwidth or FLOP rate, and the fraction of
the measured machine peaks (``MEASURED_PEAKS.json`` at the repository root when present, else the
documented fallback of 6.65 TB/s and 1.59 PFLOP/s).  ``--small`` shrinks every case to a few
launches on a few hundred MB -- the size meant for profiler captures.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
from typing import Callable, Dict

import torch

from . import QKVLayout
from . import (adamw_step, attn_varlen_bwd, attn_varlen_fwd, lmhead_logprob_fwd, paged_decode_attention,
               rmsnorm_bwd, rmsnorm_fwd, sample, swiglu_fwd)
from . import gemm as G
from . import lmhead as LM

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), "..", ".."))


def peaks() -> Dict[str, float]:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "tflops": d["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "source": "fallback"}


_flush = None


def timeit(fn: Callable[[], None], iters: int, warmup: int = 3) -> float:
    global _flush
    if _flush is None:
        _flush = (torch.empty(256 << 20, dtype=torch.uint8, device="cuda"),
                  torch.zeros(64 << 20, dtype=torch.float32, device="cuda"))
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(iters):
        # flush: write a buffer larger than L2, then read another one, so that the timed call starts with a
        # cold L2 whose lines are clean (the dirty lines of the write would otherwise be written back during
        # the timed kernel and count against its bandwidth)
        _flush[0].zero_()
        _flush[1].sum()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        # a short busy kernel ahead of the start event lets the host finish enqueueing `fn` while the
        # GPU is still occupied, so the interval holds device time only (as in a training step, where
        # launches run ahead of the GPU), not the host's launch latency
        torch.cuda._sleep(200_000)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    return statistics.median(times)


def report(name: str, ms: float, bytes_: float = 0.0, flops: float = 0.0, note: str = "") -> dict:
    pk = peaks()
    out = {"case": name, "ms": round(ms, 4)}
    if bytes_:
        gbs = bytes_ / ms / 1e6
        out.update(gbs=round(gbs, 1), frac_hbm=round(gbs / pk["hbm_gbs"], 3))
    if flops:
        tf = flops / ms / 1e9
        out.update(tflops=round(tf, 1), frac_tensor=round(tf / pk["tflops"], 3))
    out["of"] = pk["source"]
    if note:
        out["note"] = note
    print(json.dumps(out), flush=True)
    return out


def case_gemm(small: bool, iters: int):
    shapes = [(4096, 4608, 3584), (4096, 37888, 3584), (4096, 3584, 18944)] if not small else [(1024, 2048, 1024)]
    for m, n, k in shapes:
        a = torch.randn(m, k, device="cuda").bfloat16()
        b = torch.randn(n, k, device="cuda").bfloat16()
        out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
        ms = timeit(lambda: G.gemm_bf16_tn(a, b, out), iters)
        report(f"gemm_tcgen05 {m}x{n}x{k}", ms, flops=2.0 * m * n * k)
        ms = timeit(lambda: G.gemm_pair(a, b, out=out), iters)
        report(f"gemm_pair fwd   {m}x{n}x{k}", ms, flops=2.0 * m * n * k, note="cta_group::2, 256x256 tiles")
        ms = timeit(lambda: torch.matmul(a, b.t(), out=out), iters)
        report(f"gemm_cublas  {m}x{n}x{k}", ms, flops=2.0 * m * n * k, note="library baseline")
    G.check_status("cuda")


def case_gemm_pair(small: bool, iters: int):
    """The three GEMMs of a linear layer (forward, data gradient, weight gradient) on the CTA-pair
    kernel against the library calls they replace, on the 7B shapes at 8192 tokens."""
    t = 1024 if small else 8192
    layers = [("qkv", 4608, 3584), ("proj", 3584, 3584), ("fc1", 37888, 3584), ("fc2", 3584, 18944)]
    if small:
        layers = [("small", 2048, 1024)]
    for name, n, k in layers:
        x = torch.randn(t, k, device="cuda").bfloat16()
        w = (0.02 * torch.randn(n, k, device="cuda")).bfloat16()
        dy = torch.randn(t, n, device="cuda").bfloat16()
        y = torch.empty(t, n, device="cuda", dtype=torch.bfloat16)
        dx = torch.empty(t, k, device="cuda", dtype=torch.bfloat16)
        g32 = torch.zeros(n, k, device="cuda", dtype=torch.float32)
        g16 = torch.zeros(n, k, device="cuda", dtype=torch.bfloat16)
        fl = 2.0 * t * n * k
        report(f"pair fwd   {name} T={t}", timeit(lambda: G.gemm_pair(x, w, out=y), iters), flops=fl)
        report(f"cublas fwd {name} T={t}", timeit(lambda: torch.matmul(x, w.t(), out=y), iters), flops=fl)
        report(f"pair dgrad   {name} T={t}", timeit(lambda: G.gemm_pair(dy, w, b_mn=True, out=dx), iters), flops=fl)
        report(f"cublas dgrad {name} T={t}", timeit(lambda: torch.matmul(dy, w, out=dx), iters), flops=fl)
        report(f"pair wgrad(bf16 acc) {name} T={t}", timeit(lambda: G.linear_wgrad_(g16, dy, x), iters), flops=fl)
        report(f"cublas wgrad(bf16 addmm_) {name} T={t}", timeit(lambda: g16.addmm_(dy.t(), x), iters), flops=fl)
        report(f"pair wgrad(fp32 acc) {name} T={t}", timeit(lambda: G.linear_wgrad_(g32, dy, x), iters), flops=fl)
    G.check_status("cuda")


def case_gemm_pair_prof(small: bool, iters: int):
    """One mid-size forward GEMM on the CTA-pair kernel (operands and output together larger than
    L2, 8 full waves of tiles): the case meant for a profiler capture of that kernel."""
    m, n, k = 4096, 9472, 3584
    a = torch.randn(m, k, device="cuda").bfloat16()
    b = torch.randn(n, k, device="cuda").bfloat16()
    out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    report(f"gemm_pair fwd {m}x{n}x{k}", timeit(lambda: G.gemm_pair(a, b, out=out), iters, warmup=1), flops=2.0 * m * n * k)
    G.check_status("cuda")


def case_gemm_pair_ksweep(small: bool, iters: int):
    """Time of the CTA-pair kernel against the reduction length at a fixed 8-wave output: the slope
    is the main-loop rate, the intercept the fixed cost per launch and per tile."""
    m, n = 4096, 9472
    for k in (256, 512, 1024, 2048, 3584, 7168):
        a = torch.randn(m, k, device="cuda").bfloat16()
        b = torch.randn(n, k, device="cuda").bfloat16()
        out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
        report(f"gemm_pair fwd {m}x{n}x{k}", timeit(lambda: G.gemm_pair(a, b, out=out), iters), flops=2.0 * m * n * k)
        report(f"cublas    fwd {m}x{n}x{k}", timeit(lambda: torch.matmul(a, b.t(), out=out), iters), flops=2.0 * m * n * k)
    G.check_status("cuda")


def case_gemm_decode(small: bool, iters: int):
    """The four weight GEMMs of a decode step (256 tokens against the 7B layer weights): weight bytes
    streamed per second on the CTA-pair kernel and on the library call."""
    m = 256
    layers = [("qkv", 4608, 3584), ("proj", 3584, 3584), ("gate_up", 37888, 3584), ("down", 3584, 18944)]
    if small:
        layers = [("small", 4096, 1024)]
    for name, n, k in layers:
        x = torch.randn(m, k, device="cuda").bfloat16()
        w = (0.02 * torch.randn(n, k, device="cuda")).bfloat16()
        y = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
        by = 2.0 * n * k
        report(f"pair   decode {name} M={m}", timeit(lambda: G.gemm_pair(x, w, out=y), iters), bytes_=by)
        report(f"cublas decode {name} M={m}", timeit(lambda: torch.matmul(x, w.t(), out=y), iters), bytes_=by)
        plan = G.splitk_plan(m, n, k)
        for splits in sorted({plan, 4} - {0}):
            report(f"pair split-K x{splits} decode {name} M={m}" + (" (planned)" if splits == plan else ""),
                   timeit(lambda: G.gemm_pair_splitk(x, w, splits, out=y), iters), bytes_=by)
    G.check_status("cuda")


def case_fused_single(small: bool, iters: int):
    """Communication-fused GEMM variants with a team of one rank: the comm warps copy / reduce
    through local memory only, which isolates their cost from the NVLink transfer."""
    from ..parallel.fused_tp import FusedTP
    from ..parallel.symm import SymmetricArena

    m, n, k = (1024, 1024, 1024) if small else (4096, 4608, 3584)
    arena = SymmetricArena(8 * m * max(n, k) * 2 + (8 << 20))
    f = FusedTP(arena, [0], m, k, n)
    a = torch.randn(m, k, device="cuda").bfloat16()
    b = torch.randn(n, k, device="cuda").bfloat16()
    out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    report(f"gemm_tcgen05 plain      {m}x{n}x{k}", timeit(lambda: G.gemm_bf16_tn(a, b, out), iters), flops=2.0 * m * n * k)
    report(f"ag_gemm (1 rank, total) {m}x{n}x{k}", timeit(lambda: f.ag_gemm(a, b), iters), flops=2.0 * m * n * k,
           note="slot copy + barrier + memset + kernel")
    report(f"gemm_rs (1 rank)        {m}x{n}x{k}", timeit(lambda: f.gemm_rs(a, b), iters), flops=2.0 * m * n * k)
    G.check_status(a.device)
    arena.close()


def case_lmhead(small: bool, iters: int):
    t, h, v = (8192, 3584, 152064) if not small else (1024, 1024, 16384)
    x = torch.randn(t, h, device="cuda").bfloat16()
    w = (0.02 * torch.randn(v, h, device="cuda")).bfloat16()
    y = torch.randint(0, v, (t,), device="cuda")
    fl = 2.0 * t * h * v
    LM.USE_TCGEN05 = True
    ms = timeit(lambda: lmhead_logprob_fwd(x, w, y, 1.0), iters)
    report(f"lmhead_logprob fused tcgen05 T={t} V={v}", ms, flops=fl)
    LM.USE_TCGEN05 = False
    ms = timeit(lambda: lmhead_logprob_fwd(x, w, y, 1.0), iters)
    report(f"lmhead_logprob chunked cublas T={t} V={v}", ms, flops=fl, note="baseline (logits via HBM)")
    LM.USE_TCGEN05 = True
    G.check_status("cuda")


def case_attention(small: bool, iters: int):
    nh, nkv, hd = 28, 4, 128
    lay = QKVLayout(nh, nkv, hd, True)
    lens = [2048] * (8 if not small else 2)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    t = sum(lens)
    qkv = (0.5 * torch.randn(t, lay.width, device="cuda")).bfloat16()
    fl = sum(4.0 * l * l * nh * hd / 2 for l in lens)
    import os
    for flag, name in (("0", "mma.sync"), ("1", "tcgen05")):
        os.environ["MSRL_ATTN_TCGEN05"] = flag
        out, lse = attn_varlen_fwd(qkv, lay, cu, max(lens))
        ms = timeit(lambda: attn_varlen_fwd(qkv, lay, cu, max(lens)), iters)
        report(f"flash_attn_varlen fwd {name} T={t}", ms, flops=fl)
    G.check_status("cuda", "tcgen05 attention")
    do = torch.randn_like(out)
    for flag, name in (("0", "mma.sync"), ("1", "tcgen05")):
        os.environ["MSRL_ATTN_TCGEN05"] = flag
        ms = timeit(lambda: attn_varlen_bwd(do, qkv, out, lse, lay, cu, max(lens)), iters)
        report(f"flash_attn_varlen bwd {name} T={t}", ms, flops=2.5 * fl)
    G.check_status("cuda", "tcgen05 attention")


def case_decode(small: bool, iters: int):
    nh, nkv, hd, bs = 28, 4, 128, 16
    lay = QKVLayout(nh, nkv, hd, True)
    b, ctx = (256, 2048) if not small else (32, 1024)
    nblk = b * ctx // bs
    kc = torch.randn(nblk, bs, nkv, hd, device="cuda").bfloat16()
    vc = torch.randn(nblk, bs, nkv, hd, device="cuda").bfloat16()
    bt = torch.randperm(nblk, device="cuda").to(torch.int32).view(b, ctx // bs)
    cl = torch.full((b,), ctx, dtype=torch.int32, device="cuda")
    q = torch.randn(b, lay.width, device="cuda").bfloat16()
    ms = timeit(lambda: paged_decode_attention(q, lay, kc, vc, bt, cl, ctx), iters)
    report(f"paged_decode B={b} ctx={ctx}", ms, bytes_=2.0 * b * ctx * nkv * hd * 2)
    # n-sample groups: 8 samples share a 1024-token prompt (same physical blocks), 1024 own tokens each
    from .decode import build_decode_groups, decode_group_max

    n, prompt = 8, 1024
    shared = prompt // bs
    bt2 = bt.clone()
    for g in range(b // n):
        bt2[g * n:(g + 1) * n, :shared] = bt[g * n, :shared]
    from .decode import decode_prefix_tile

    tile = decode_prefix_tile(nh, nkv, hd, bs)
    ks, rows, pre, _ = build_decode_groups([i // n for i in range(b)], [prompt] * b, decode_group_max(nh, nkv, tile),
                                           multiple=max(1, tile))
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    real = sum(1 for r in rows if r[0] >= 0)
    groups = (i32(ks), i32(rows[:real]), i32(pre[:real]))
    unique_bytes = 2.0 * (b // n * prompt + b * (ctx - prompt)) * nkv * hd * 2
    ms_plain = timeit(lambda: paged_decode_attention(q, lay, kc, vc, bt2, cl, ctx), iters)
    report(f"paged_decode shared-prompt layout, plain kernel B={b}", ms_plain, bytes_=2.0 * b * ctx * nkv * hd * 2,
           note="every sample re-reads the shared prompt")
    ms = timeit(lambda: paged_decode_attention(q, lay, kc, vc, bt2, cl, ctx, groups=groups, prefix_tile=tile), iters)
    report(f"paged_decode shared-prefix kernels B={b} (8 x 1024 shared + 1024 own)", ms, bytes_=unique_bytes,
           note=f"unique K/V bytes; {ms_plain / ms:.2f}x faster than the plain kernel on the same cache")


def case_decode_prefix(small: bool, iters: int):
    """Shared-prefix decode with short own suffixes, so that the prefix pass dominates: sweep of the
    number of prefix splits per (group, KV head)."""
    from .decode import build_decode_groups, decode_group_max, decode_prefix_tile

    nh, nkv, hd, bs = 28, 4, 128, 16
    lay = QKVLayout(nh, nkv, hd, True)
    b, n, prompt = (256, 8, 1024) if not small else (64, 8, 1024)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    q = torch.randn(b, lay.width, device="cuda").bfloat16()
    for own in (16, 512):
        ctx = prompt + own
        per = (ctx + bs - 1) // bs
        nblk = b * per
        kc = torch.randn(nblk, bs, nkv, hd, device="cuda").bfloat16()
        vc = torch.randn(nblk, bs, nkv, hd, device="cuda").bfloat16()
        bt = torch.randperm(nblk, device="cuda").to(torch.int32).view(b, per)
        shared = prompt // bs
        for g in range(b // n):
            bt[g * n:(g + 1) * n, :shared] = bt[g * n, :shared].clone()
        cl = torch.full((b,), ctx, dtype=torch.int32, device="cuda")
        unique = 2.0 * (b // n * prompt + b * own) * nkv * hd * 2
        for tile in sorted({0, decode_prefix_tile(nh, nkv, hd, bs)}):
            ks, rows, pre, _ = build_decode_groups([i // n for i in range(b)], [prompt] * b,
                                                   decode_group_max(nh, nkv, tile), multiple=max(1, tile))
            real = sum(1 for r in rows if r[0] >= 0)
            groups = (i32(ks), i32(rows[:real]), i32(pre[:real]))
            kind = "tcgen05" if tile else "mma.sync"
            for splits in (1, 2, 4, 8):
                ms = timeit(lambda: paged_decode_attention(q, lay, kc, vc, bt, cl, ctx, groups=groups,
                                                           prefix_splits=splits, prefix_tile=tile), iters)
                report(f"paged_decode grouped ({kind} prefix pass) B={b} prompt={prompt} own={own} "
                       f"prefix_splits={splits}", ms, bytes_=unique)


def case_elementwise(small: bool, iters: int):
    rows, h, f = (16384, 3584, 18944) if not small else (4096, 3584, 4096)
    x = torch.randn(rows, h, device="cuda").bfloat16()
    w = torch.ones(h, device="cuda").bfloat16()
    ms = timeit(lambda: rmsnorm_fwd(x, w, 1e-6), iters)
    report(f"rmsnorm fwd {rows}x{h}", ms, bytes_=2.0 * rows * h * 2)
    y, rstd, _ = rmsnorm_fwd(x, w, 1e-6)
    dw = torch.zeros(h, device="cuda")
    ms = timeit(lambda: rmsnorm_bwd(x, x, w, rstd, dw), iters)
    report(f"rmsnorm bwd {rows}x{h}", ms, bytes_=3.0 * rows * h * 2)
    gu = torch.randn(rows, 2 * f, device="cuda").bfloat16()
    ms = timeit(lambda: swiglu_fwd(gu), iters)
    report(f"swiglu fwd {rows}x{f}", ms, bytes_=3.0 * rows * f * 2)


def case_adam(small: bool, iters: int):
    n = (1 << 30) // 4 if not small else (1 << 26)
    p = torch.randn(n, device="cuda")
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    g = torch.randn(n, device="cuda").bfloat16()
    p16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    ms = timeit(lambda: adamw_step(p, m, v, g, p16, 1e-6, 0.9, 0.95, 1e-8, 0.01, 1), iters)
    report(f"adamw n={n}", ms, bytes_=n * (3 * 4 * 2 + 2 + 2))


def case_sampler(small: bool, iters: int):
    b, v = (256, 152064) if not small else (64, 32768)
    logits = torch.randn(b, v, device="cuda").bfloat16()
    t = torch.ones(b, device="cuda")
    keys = torch.arange(b, device="cuda", dtype=torch.int64)
    ms = timeit(lambda: sample(logits, t, None, None, None, keys, 0), iters)
    report(f"sampler B={b} V={v}", ms, bytes_=2.0 * b * v * 2, note="two passes over the logits")


def case_moe(small: bool, iters: int):
    """Qwen3-30B-A3B expert shapes on one expert-parallel rank: 16 local experts, hidden 2048,
    expert FFN 768, top-8 routing."""
    from . import moe as K
    from . import swiglu_fwd
    e, h, f, k = 16, 2048, 768, 8
    t = 2048 if small else 16384
    x = torch.randn(t, h, device="cuda").bfloat16()
    idx = torch.stack([torch.randperm(e, device="cuda")[:k] for _ in range(256)]).repeat(t // 256, 1)
    p = torch.rand(t, k, device="cuda")
    w1 = (torch.randn(h, e, 2 * f, device="cuda") * 0.02).bfloat16()
    w2 = (torch.randn(e, f, h, device="cuda") * 0.02).bfloat16()
    w1_2d, w2_2d = w1.view(h, e * 2 * f), w2.view(e * f, h)
    plan = K.moe_plan(idx, e)
    ms = timeit(lambda: K.moe_plan(idx, e), iters)
    report(f"moe_plan slots={t * k} E={e}", ms, bytes_=t * k * 12.0)
    xp = K.moe_permute(x, plan)
    ms = timeit(lambda: K.moe_permute(x, plan), iters)
    report(f"moe_permute T={t} k={k} H={h}", ms, bytes_=(t + t * k) * h * 2.0)
    rows = t * k
    gu = K.grouped_gemm(xp, plan, w1_2d, True, 2 * f, 0, 2 * f)
    ms = timeit(lambda: K.grouped_gemm(xp, plan, w1_2d, True, 2 * f, 0, 2 * f), iters)
    report(f"grouped_gemm w1 (MN-major B) rows={rows}", ms, flops=2.0 * rows * h * 2 * f)
    act = swiglu_fwd(gu)
    y = K.grouped_gemm(act, plan, w2_2d, True, 0, f, h)
    ms = timeit(lambda: K.grouped_gemm(act, plan, w2_2d, True, 0, f, h), iters)
    report(f"grouped_gemm w2 (MN-major B) rows={rows}", ms, flops=2.0 * rows * f * h)
    ms = timeit(lambda: K.grouped_gemm(y, plan, w2_2d, False, 0, f, f), iters)
    report(f"grouped_gemm dact (K-major B) rows={rows}", ms, flops=2.0 * rows * f * h)
    counts, offsets = plan.counts.tolist(), plan.offsets.tolist()

    def loop():
        for j, n in enumerate(counts):
            torch.matmul(xp[offsets[j]:offsets[j] + n], w1[:, j], out=gu[offsets[j]:offsets[j] + n])
    ms = timeit(loop, iters)
    report(f"per-expert cuBLAS loop w1 rows={rows}", ms, flops=2.0 * rows * h * 2 * f, note="baseline")
    ms = timeit(lambda: K.moe_combine(y, plan, p), iters)
    report(f"moe_combine T={t} k={k} H={h}", ms, bytes_=(t + t * k) * h * 2.0)
    G.check_status("cuda", "grouped gemm")


CASES = {"moe": case_moe, "gemm": case_gemm, "gemm_pair": case_gemm_pair, "gemm_pair_prof": case_gemm_pair_prof, "gemm_pair_ksweep": case_gemm_pair_ksweep, "gemm_decode": case_gemm_decode, "lmhead": case_lmhead, "attention": case_attention, "decode": case_decode, "decode_prefix": case_decode_prefix,
         "elementwise": case_elementwise, "adam": case_adam, "sampler": case_sampler,
         "fused_single": case_fused_single}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="")
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    names = [n for n in args.only.split(",") if n] or list(CASES)
    for n in names:
        CASES[n](args.small, args.iters)


if __name__ == "__main__":
    main()
