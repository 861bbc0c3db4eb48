"""Mixture-of-experts token movement and grouped expert GEMMs.

``moe_plan`` turns the expert id of every (token, k) slot into a dispatch plan (per-expert counts,
128-row padded segment offsets, destination row per slot, expert per 128-row tile) without a host
round trip; ``moe_permute`` / ``moe_combine`` / ``moe_slot_dot`` move rows along it;
``grouped_gemm`` multiplies every row tile with its expert's weight on the tcgen05 tensor cores,
reading the weights in place (K-major or MN-major operand) from one 2-D view of the stacked
parameter.  CUDA path: ``csrc/moe.cu``, ``csrc/moe_gemm_tcgen05.cu``; CPU tensors run the PyTorch
formulation that is also the test oracle.  Reference behaviour:
``mindspeed_rl/models/rollout/vllm_adapter/fused_moe.py:55-373``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import guard

from . import _lib
from ._lib import c_int, c_ll, check, ptr, stream

PAD = 128
_NOT_SUPPORTED = 801


@dataclass
class MoePlan:
    counts: torch.Tensor        # [E] int32 rows per expert
    offsets: torch.Tensor       # [E+1] int32 first row of every (padded) segment
    pos: torch.Tensor           # [T*k] int32 destination row of every slot
    tile_expert: torch.Tensor   # [max_rows/128] int32, -1 = tile not in use
    max_rows: int               # rows of the expert-grouped buffers (host-side bound)
    tokens: int
    k: int
    num_experts: int


def max_rows(n_slots: int, num_experts: int) -> int:
    """Upper bound on the padded row count that needs no look at the routing result."""
    return (n_slots + PAD - 1) // PAD * PAD + num_experts * PAD


def moe_plan(expert_of: torch.Tensor, num_experts: int) -> MoePlan:
    """``expert_of [T, k]`` (int64) -> :class:`MoePlan`; slots of an expert keep their order."""
    t, k = expert_of.shape
    n = t * k
    rows = max_rows(n, num_experts)
    dev = expert_of.device
    flat = expert_of.reshape(-1).contiguous()
    if _lib.use_kernels(expert_of):
        counts = guard.empty(num_experts, dtype=torch.int32, device=dev)
        offsets = guard.empty(num_experts + 1, dtype=torch.int32, device=dev)
        pos = guard.empty(n, dtype=torch.int32, device=dev)
        tiles = guard.empty(rows // PAD, dtype=torch.int32, device=dev)
        blocks = (n + 255) // 256
        scratch = guard.empty(blocks * num_experts + n + 1, dtype=torch.int32, device=dev)
        check(_lib.load().msrl_moe_plan(ptr(flat), c_int(n), c_int(num_experts), ptr(scratch), ptr(counts),
                                        ptr(offsets), ptr(pos), ptr(tiles), c_int(rows // PAD), stream()), "moe_plan")
        return MoePlan(counts, offsets, pos, tiles, rows, t, k, num_experts)
    counts = torch.bincount(flat, minlength=num_experts)
    padded = (counts + PAD - 1) // PAD * PAD
    offsets = torch.zeros(num_experts + 1, dtype=torch.int64, device=dev)
    offsets[1:] = padded.cumsum(0)
    order = torch.argsort(flat, stable=True)
    rank = guard.empty(n, dtype=torch.int64, device=dev)
    start = counts.cumsum(0) - counts
    rank[order] = torch.arange(n, device=dev) - start[flat[order]]
    pos = offsets[flat] + rank
    tiles = torch.full((rows // PAD,), -1, dtype=torch.int32, device=dev)
    for e in range(num_experts):
        tiles[int(offsets[e]) // PAD:int(offsets[e + 1]) // PAD] = e
    return MoePlan(counts.int(), offsets.int(), pos.int(), tiles, rows, t, k, num_experts)


def moe_permute(x: torch.Tensor, plan: MoePlan, w: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x [T, H]`` -> expert-grouped ``[max_rows, H]`` (row of slot (t, j) = ``w[t, j] * x[t]``);
    pad rows of used segments are zero, rows past the last segment are not touched."""
    t, h = x.shape
    if _lib.use_kernels(x):
        x = x.contiguous()
        xp = guard.empty(plan.max_rows, h, dtype=x.dtype, device=x.device)
        wf = None if w is None else w.reshape(-1).float().contiguous()
        check(_lib.load().msrl_moe_permute(ptr(x), c_ll(h), ptr(plan.pos), ptr(wf), c_int(t), c_int(plan.k), c_int(h),
                                           c_int(plan.num_experts), ptr(plan.counts), ptr(plan.offsets), ptr(xp),
                                           c_ll(h), stream()), "moe_permute")
        return xp
    xp = torch.zeros(plan.max_rows, h, dtype=x.dtype, device=x.device)
    rows = x.repeat_interleave(plan.k, dim=0)
    if w is not None:
        rows = (rows.float() * w.reshape(-1, 1).float()).to(x.dtype)
    xp[plan.pos.long()] = rows
    return xp


def moe_combine(y: torch.Tensor, plan: MoePlan, w: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[t] = sum_j w[t, j] * y[pos(t, j)]`` (fp32 accumulation), ``[T, H]`` in ``y``'s dtype."""
    h = y.shape[1]
    if _lib.use_kernels(y):
        out = guard.empty(plan.tokens, h, dtype=y.dtype, device=y.device)
        wf = None if w is None else w.reshape(-1).float().contiguous()
        check(_lib.load().msrl_moe_combine(ptr(y), c_ll(y.stride(0)), ptr(plan.pos), ptr(wf), c_int(plan.tokens),
                                           c_int(plan.k), c_int(h), ptr(out), c_ll(h), c_int(0), stream()),
              "moe_combine")
        return out
    rows = y[plan.pos.long()].float().view(plan.tokens, plan.k, h)
    if w is not None:
        rows = rows * w.float().view(plan.tokens, plan.k, 1)
    return rows.sum(1).to(y.dtype)


def moe_slot_dot(dout: torch.Tensor, y: torch.Tensor, plan: MoePlan) -> torch.Tensor:
    """``dw[t, j] = <dout[t], y[pos(t, j)]>`` (fp32): gradient of the combine weights."""
    h = y.shape[1]
    if _lib.use_kernels(dout, y):
        dout = dout.contiguous()
        dw = guard.empty(plan.tokens, plan.k, dtype=torch.float32, device=y.device)
        check(_lib.load().msrl_moe_slot_dot(ptr(dout), c_ll(h), ptr(y), c_ll(y.stride(0)), ptr(plan.pos),
                                            c_int(plan.tokens), c_int(plan.k), c_int(h), ptr(dw), stream()),
              "moe_slot_dot")
        return dw
    rows = y[plan.pos.long()].float().view(plan.tokens, plan.k, h)
    return (rows * dout.float().unsqueeze(1)).sum(-1)


def _sm_count(device) -> int:
    return torch.cuda.get_device_properties(device).multi_processor_count


def grouped_wgrad_(grad: torch.Tensor, group_stride: int, ldc: int, a: torch.Tensor, b: torch.Tensor,
                   plan: MoePlan) -> bool:
    """``grad_e[M, N] += a[rows of e].T @ b[rows of e]`` for every expert e of ``plan`` in ONE launch of the
    CTA-pair GEMM (``csrc/gemm2cta_tcgen05.cu``, grouped reduction): ``a [rows, M]`` and ``b [rows, N]`` are
    permuted-layout activations whose pad rows are zero, ``grad`` is a view whose first element is expert 0's
    block; expert ``e``'s block starts ``group_stride`` elements later and has leading dimension ``ldc``.
    The segment bounds are read on the device (``plan.offsets``): no host round trip.  Returns ``False``
    (nothing done) for inputs the kernel does not cover; the caller then loops over the experts."""
    from .gemm import _status_word, pair_enabled, pair_usable

    if not (a.is_cuda and pair_enabled() and pair_usable(a, b) and _lib.use_kernels(a, b, grad)
            and grad.dtype in (torch.float32, torch.bfloat16) and grad.data_ptr() % 16 == 0
            and ldc % 8 == 0 and group_stride % 8 == 0 and a.shape[0] == b.shape[0] and a.shape[0] % 8 == 0
            and plan.offsets is not None and plan.offsets.dtype == torch.int32):
        return False
    groups = int(plan.offsets.numel()) - 1
    check(_lib.load().msrl_gemm_pair_grouped_wgrad(
        ptr(a), c_ll(a.stride(0)), ptr(b), c_ll(b.stride(0)), ptr(grad), c_ll(ldc), c_ll(group_stride),
        c_int(1 if grad.dtype == torch.float32 else 2), ptr(plan.offsets), c_int(groups), c_int(a.shape[1]),
        c_int(b.shape[1]), c_ll(a.shape[0]), ptr(_status_word(a.device)), stream()), "gemm_pair_grouped_wgrad")
    return True


def grouped_gemm(a: torch.Tensor, plan: MoePlan, b2d: torch.Tensor, b_mn_major: bool, ex: int, ey: int,
                 n: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``c[r] = a[r] @ B_e`` for the rows of expert e.  ``b2d`` is a 2-D contiguous view of all
    experts' weights; expert e's operand starts at ``b2d[e*ey, e*ex]`` and is ``[K, n]`` when
    ``b_mn_major`` else ``[n, K]`` (used transposed).  Rows of ``c`` outside used tiles are
    undefined; pad rows inside used tiles are the product of zero rows."""
    rows, k = a.shape
    if _lib.use_kernels(a, b2d):
        from .gemm import _status_word
        assert a.is_contiguous() and b2d.is_contiguous() and rows == plan.max_rows
        c = guard.empty(rows, n, dtype=a.dtype, device=a.device) if out is None else out
        assert c.shape == (rows, n) and c.is_contiguous()
        rc = _lib.load().msrl_moe_grouped_gemm(
            ptr(a), c_ll(k), ptr(b2d), c_ll(b2d.shape[0]), c_ll(b2d.shape[1]), c_ll(b2d.shape[1]),
            c_int(1 if b_mn_major else 0), c_int(ex), c_int(ey), ptr(c), c_ll(n), ptr(plan.tile_expert),
            c_int(rows // PAD), c_int(n), c_int(k), c_int(_sm_count(a.device)), ptr(_status_word(a.device)), stream())
        if rc != _NOT_SUPPORTED:
            check(rc, "moe_grouped_gemm")
            return c
    c = torch.zeros(rows, n, dtype=a.dtype, device=a.device) if out is None else out.zero_()
    counts, offsets = plan.counts.tolist(), plan.offsets.tolist()
    for e, cnt in enumerate(counts):
        if cnt == 0:
            continue
        r0 = offsets[e]
        if b_mn_major:
            be = b2d[e * ey:e * ey + k, e * ex:e * ex + n]
            torch.matmul(a[r0:r0 + cnt], be, out=c[r0:r0 + cnt])
        else:
            be = b2d[e * ey:e * ey + n, e * ex:e * ex + k]
            torch.matmul(a[r0:r0 + cnt], be.t(), out=c[r0:r0 + cnt])
    return c
