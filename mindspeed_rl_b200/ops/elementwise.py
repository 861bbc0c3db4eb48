"""RMSNorm / per-head norm / RoPE / SwiGLU / bias-grad front-ends.

Every function has explicit forward and backward entry points (the transformer layer calls
them by hand inside one autograd node and accumulates parameter gradients in place).  CUDA
tensors go to the sm_100a kernels in ``csrc/elementwise.cu``; CPU tensors use the fp32
PyTorch formulation that doubles as the numerics oracle in the tests.
"""
from __future__ import annotations

from functools import lru_cache
from typing import Optional, Tuple

import torch

from . import guard

from . import _lib
from ._lib import c_float, c_int, c_ll, check, ptr, stream
from .layouts import QKVLayout

_scratch = {}
_retired = []     # outgrown scratch buffers stay allocated: captured CUDA graphs may still point at them


def _workspace(key: str, numel: int, device, dtype=torch.float32) -> torch.Tensor:
    """Grow-only scratch buffers (kernels never allocate)."""
    buf = _scratch.get((key, device, dtype))
    if buf is None or buf.numel() < numel:
        if buf is not None and buf.is_cuda:
            _retired.append(buf)
        buf = guard.empty(max(numel, 1), device=device, dtype=dtype)
        _scratch[(key, device, dtype)] = buf
    return buf


# ------------------------------------------------------------------------------------------------
# RMSNorm
# ------------------------------------------------------------------------------------------------
def rmsnorm_fwd(x: torch.Tensor, w: torch.Tensor, eps: float, residual: Optional[torch.Tensor] = None,
                want_rstd: bool = True) -> Tuple[torch.Tensor, Optional[torch.Tensor], Optional[torch.Tensor]]:
    """``y = (x [+ residual]) * rsqrt(mean(.^2) + eps) * w``.

    Returns ``(y, rstd, summed)`` where ``summed`` is ``x + residual`` (``None`` without residual).
    """
    h = x.shape[-1]
    rows = x.numel() // h
    if _lib.use_kernels(x, w):
        x2 = x.contiguous().view(rows, h)
        y = guard.empty_like(x2)
        rstd = guard.empty(rows, device=x.device, dtype=torch.float32) if want_rstd else None
        summed = guard.empty_like(x2) if residual is not None else None
        res = residual.contiguous().view(rows, h) if residual is not None else None
        check(_lib.load().msrl_rmsnorm_fwd(ptr(x2), ptr(res), ptr(w), ptr(y), ptr(summed), ptr(rstd),
                                           c_ll(rows), c_int(h), c_float(eps), stream()),
              "rmsnorm_fwd")
        return (y.view_as(x), rstd, summed.view_as(x) if summed is not None else None)
    xs = x if residual is None else (x.float() + residual.float()).to(x.dtype)
    xf = xs.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    y = (xf * rstd * w.float()).to(x.dtype)
    return y, (rstd.reshape(rows) if want_rstd else None), (xs if residual is not None else None)


def rmsnorm_bwd(dy: torch.Tensor, x: torch.Tensor, w: torch.Tensor, rstd: torch.Tensor,
                dw_accum: torch.Tensor, dres: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Returns ``dx (+ dres)`` and adds the weight gradient into ``dw_accum`` (fp32 or bf16)."""
    h = x.shape[-1]
    rows = x.numel() // h
    if _lib.use_kernels(dy, x, w):
        L = _lib.load()
        dy2, x2 = dy.contiguous().view(rows, h), x.contiguous().view(rows, h)
        dx = guard.empty_like(x2)
        nb = L.msrl_rmsnorm_bwd_blocks(c_ll(rows))
        part = _workspace("rmsnorm_dw", nb * h, x.device)
        dres2 = dres.contiguous().view(rows, h) if dres is not None else None
        f32 = dw_accum.dtype == torch.float32
        check(L.msrl_rmsnorm_bwd(ptr(dy2), ptr(x2), ptr(w), ptr(rstd), ptr(dres2), ptr(dx), ptr(part),
                                 ptr(dw_accum) if f32 else None, None if f32 else ptr(dw_accum),
                                 c_int(1), c_ll(rows), c_int(h), stream()), "rmsnorm_bwd")
        return dx.view_as(x)
    xf, dyf = x.float().view(rows, h), dy.float().view(rows, h)
    rs = rstd.view(rows, 1).float()
    g = dyf * w.float()
    dot = (g * xf).sum(-1, keepdim=True)
    dx = g * rs - xf * (dot * rs.pow(3) / h)
    dw_accum.add_((dyf * xf * rs).sum(0).to(dw_accum.dtype))
    if dres is not None:
        dx = dx + dres.float().view(rows, h)
    return dx.to(x.dtype).view_as(x)


# ------------------------------------------------------------------------------------------------
# Per-head RMSNorm on the q / k heads of a fused QKV tensor (QK-norm), in place
# ------------------------------------------------------------------------------------------------
def _head_spec(layout: QKVLayout, which: str):
    return {"q": layout.q, "k": layout.k, "v": layout.v}[which]()


def _nheads(layout: QKVLayout, which: str) -> int:
    return layout.num_heads if which == "q" else layout.num_kv_heads


def headnorm_fwd_(qkv: torch.Tensor, layout: QKVLayout, which: str, w: torch.Tensor, eps: float
                  ) -> torch.Tensor:
    """Normalise every ``which`` head of ``qkv`` in place; returns rstd ``[T * nheads]``.

    The caller keeps a copy of the un-normalised heads when it needs the backward.
    """
    t = qkv.shape[0]
    n = _nheads(layout, which)
    hd = layout.head_dim
    off, (st, gs, hpg, hs) = _head_spec(layout, which)
    if _lib.use_kernels(qkv, w):
        rstd = guard.empty(t * n, device=qkv.device, dtype=torch.float32)
        base = qkv.view(-1)[off:]
        check(_lib.load().msrl_headnorm_fwd(ptr(base), c_ll(st), c_int(gs), c_int(hpg), c_int(hs), ptr(w),
                                            ptr(base), ptr(rstd), c_ll(t), c_int(n), c_int(hd),
                                            c_float(eps), stream()), "headnorm_fwd")
        return rstd
    q, k, v = layout.split(qkv)
    src = q if which == "q" else k
    xf = src.float()
    rs = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    out = (xf * rs * w.float()).to(qkv.dtype)
    parts = dict(q=q, k=k, v=v)
    parts[which] = out
    qkv.copy_(layout.merge(parts["q"], parts["k"], parts["v"]))
    return rs.reshape(t * n)


def headnorm_bwd_(dqkv: torch.Tensor, qkv_pre: torch.Tensor, layout: QKVLayout, which: str,
                  w: torch.Tensor, rstd: torch.Tensor, dw_accum: torch.Tensor) -> None:
    """In place on ``dqkv``: gradient w.r.t. the un-normalised heads; ``qkv_pre`` holds them."""
    t = dqkv.shape[0]
    n = _nheads(layout, which)
    hd = layout.head_dim
    off, (st, gs, hpg, hs) = _head_spec(layout, which)
    if _lib.use_kernels(dqkv, qkv_pre, w):
        L = _lib.load()
        nb = L.msrl_headnorm_bwd_blocks()
        part = _workspace("headnorm_dw", nb * hd, dqkv.device)
        f32 = dw_accum.dtype == torch.float32
        check(L.msrl_headnorm_bwd(ptr(dqkv.view(-1)[off:]), ptr(qkv_pre.view(-1)[off:]), c_ll(st),
                                  c_int(gs), c_int(hpg), c_int(hs), ptr(w), ptr(rstd), ptr(part),
                                  ptr(dw_accum) if f32 else None, None if f32 else ptr(dw_accum),
                                  c_int(1), c_ll(t), c_int(n), c_int(hd), stream()), "headnorm_bwd")
        return
    dq, dk, dv = layout.split(dqkv)
    q, k, _ = layout.split(qkv_pre)
    d, x = (dq, q) if which == "q" else (dk, k)
    df, xf = d.float(), x.float()
    rs = rstd.view(t, n, 1).float()
    g = df * w.float()
    dot = (g * xf).sum(-1, keepdim=True)
    dx = (g * rs - xf * (dot * rs.pow(3) / hd)).to(dqkv.dtype)
    dw_accum.add_((df * xf * rs).sum((0, 1)).to(dw_accum.dtype))
    parts = dict(q=dq, k=dk, v=dv)
    parts[which] = dx
    dqkv.copy_(layout.merge(parts["q"], parts["k"], parts["v"]))


# ------------------------------------------------------------------------------------------------
# RoPE
# ------------------------------------------------------------------------------------------------
@lru_cache(maxsize=16)
def _rope_table_cpu(max_pos: int, head_dim: int, theta: float, scaling_key=None) -> torch.Tensor:
    half = head_dim // 2
    inv = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float64) * 2.0 / head_dim))
    mscale = 1.0
    if scaling_key is not None:
        inv, mscale = _yarn_inv_freq(inv, head_dim, theta, dict(scaling_key))
    ang = torch.arange(max_pos, dtype=torch.float64).unsqueeze(1) * inv.unsqueeze(0)
    return torch.cat([ang.cos() * mscale, ang.sin() * mscale], dim=1).float().contiguous()


def _yarn_inv_freq(inv, head_dim, theta, sc):
    """YaRN frequency interpolation (``rope_scaling_type: yarn``)."""
    import math

    factor = float(sc.get("factor", 1.0))
    orig = float(sc.get("original_max_position_embeddings", 4096))
    beta_fast, beta_slow = float(sc.get("beta_fast", 32)), float(sc.get("beta_slow", 1))

    def corr_dim(rot):
        return head_dim * math.log(orig / (rot * 2 * math.pi)) / (2 * math.log(theta))

    lo = max(math.floor(corr_dim(beta_fast)), 0)
    hi = min(math.ceil(corr_dim(beta_slow)), head_dim // 2 - 1)
    ramp = ((torch.arange(head_dim // 2, dtype=torch.float64) - lo) / max(hi - lo, 1e-3)).clamp(0, 1)
    mask = 1.0 - ramp
    inv_new = inv / factor * (1 - mask) + inv * mask

    def get_mscale(scale, m):
        return 1.0 if scale <= 1 else 0.1 * m * math.log(scale) + 1.0

    m = float(sc.get("mscale", 1.0))
    m_all = float(sc.get("mscale_all_dim", 0.0))
    mscale = get_mscale(factor, m) / get_mscale(factor, m_all) if m_all else get_mscale(factor, m)
    return inv_new, mscale


_rope_dev_cache = {}


def rope_table(max_pos: int, head_dim: int, theta: float, device, scaling: Optional[dict] = None
               ) -> torch.Tensor:
    """``[max_pos, head_dim]`` fp32 table ``[cos | sin]`` (rotate-half pairing)."""
    key = (max_pos, head_dim, float(theta), tuple(sorted(scaling.items())) if scaling else None,
           str(device))
    tab = _rope_dev_cache.get(key)
    if tab is None:
        tab = _rope_table_cpu(key[0], key[1], key[2], key[3]).to(device)
        _rope_dev_cache[key] = tab
    return tab


def rope_(qkv: torch.Tensor, layout: QKVLayout, positions: torch.Tensor, table: torch.Tensor,
          inverse: bool = False) -> torch.Tensor:
    """Rotate the q and k heads of ``qkv`` in place (``inverse=True`` is the backward)."""
    t = qkv.shape[0]
    hd = layout.head_dim
    if _lib.use_kernels(qkv, positions, table):
        qo, (qs, qg, qh, qhs) = layout.q()
        ko, (ks, kg, kh, khs) = layout.k()
        flat = qkv.view(-1)
        pos = positions if positions.dtype == torch.int32 else positions.to(torch.int32)
        check(_lib.load().msrl_rope(ptr(flat[qo:]), c_ll(qs), c_int(qg), c_int(qh), c_int(qhs),
                                    c_int(layout.num_heads), ptr(flat[ko:]), c_ll(ks), c_int(kg),
                                    c_int(kh), c_int(khs), c_int(layout.num_kv_heads), ptr(pos),
                                    ptr(table), c_ll(t), c_int(hd), c_float(-1.0 if inverse else 1.0),
                                    stream()), "rope")
        return qkv
    q, k, v = layout.split(qkv)
    cs = table[positions.long()]
    cos, sin = cs[:, None, :hd // 2], cs[:, None, hd // 2:]
    if inverse:
        sin = -sin

    def rot(x):
        xf = x.float()
        a, b = xf[..., :hd // 2], xf[..., hd // 2:]
        return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1).to(x.dtype)

    qkv.copy_(layout.merge(rot(q), rot(k), v))
    return qkv


# ------------------------------------------------------------------------------------------------
# SwiGLU
# ------------------------------------------------------------------------------------------------
def swiglu_fwd(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``silu(gate) * up`` of ``[..., gate | up]``; ``out`` (contiguous, ``[..., F]``) receives the result."""
    f = gate_up.shape[-1] // 2
    rows = gate_up.numel() // (2 * f)
    if _lib.use_kernels(gate_up):
        x = gate_up.contiguous()
        if out is None:
            out = guard.empty(*x.shape[:-1], f, device=x.device, dtype=x.dtype)
        check(_lib.load().msrl_swiglu_fwd(ptr(x), ptr(out), c_ll(rows), c_int(f), stream()), "swiglu_fwd")
        return out
    g, u = gate_up.float().split(f, dim=-1)
    y = (torch.nn.functional.silu(g) * u).to(gate_up.dtype)
    return y if out is None else out.copy_(y)


def swiglu_bwd(gate_up: torch.Tensor, dy: torch.Tensor) -> torch.Tensor:
    f = gate_up.shape[-1] // 2
    rows = gate_up.numel() // (2 * f)
    if _lib.use_kernels(gate_up, dy):
        x, d = gate_up.contiguous(), dy.contiguous()
        out = guard.empty_like(x)
        check(_lib.load().msrl_swiglu_bwd(ptr(x), ptr(d), ptr(out), c_ll(rows), c_int(f), stream()),
              "swiglu_bwd")
        return out
    g, u = gate_up.float().split(f, dim=-1)
    s = torch.sigmoid(g)
    d = dy.float()
    return torch.cat([d * u * s * (1 + g * (1 - s)), d * g * s], dim=-1).to(gate_up.dtype)


# ------------------------------------------------------------------------------------------------
# misc
# ------------------------------------------------------------------------------------------------
def colsum_accumulate(m: torch.Tensor, out: torch.Tensor) -> None:
    """``out += m.sum(0)`` for a 2-D bf16 ``m`` (bias gradients)."""
    rows, c = m.shape
    if _lib.use_kernels(m, out) and m.dtype == torch.bfloat16:
        L = _lib.load()
        part = _workspace("colsum", L.msrl_colsum_blocks() * c, m.device)
        f32 = out.dtype == torch.float32
        check(L.msrl_colsum(ptr(m.contiguous()), c_ll(rows), c_int(c), ptr(part),
                            ptr(out) if f32 else None, None if f32 else ptr(out), c_int(1), stream()),
              "colsum")
        return
    out.add_(m.float().sum(0).to(out.dtype))


def add(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    if _lib.use_kernels(a, b) and a.dtype == torch.bfloat16 and a.numel() % 8 == 0 \
            and a.is_contiguous() and b.is_contiguous():
        out = guard.empty_like(a)
        check(_lib.load().msrl_add(ptr(a), ptr(b), ptr(out), c_ll(a.numel()), stream()), "add")
        return out
    return a + b


def embedding_grad_(g: torch.Tensor, d: torch.Tensor, order: torch.Tensor, uniq: torch.Tensor,
                    counts: torch.Tensor) -> bool:
    """``g[uniq[s]] += sum of d[order[t]]`` over segment ``s`` of the id-sorted tokens (``counts[s]`` tokens
    each), rows of one id added in fp32 in token order.  Returns ``False`` (nothing done) when the kernel
    does not cover the inputs; the caller then takes the PyTorch formulation."""
    if not (_lib.use_kernels(g, d) and d.dtype == torch.bfloat16 and g.dtype in (torch.bfloat16, torch.float32)
            and d.dim() == 2 and g.dim() == 2 and d.stride(1) == 1 and g.stride(1) == 1 and d.shape[1] % 8 == 0
            and d.stride(0) % 8 == 0 and g.stride(0) % 8 == 0 and d.data_ptr() % 16 == 0 and g.data_ptr() % 16 == 0):
        return False
    n_seg = int(uniq.numel())
    seg_start = torch.zeros(n_seg + 1, dtype=torch.int64, device=d.device)
    torch.cumsum(counts, 0, out=seg_start[1:])
    check(_lib.load().msrl_embedding_grad(ptr(d), c_ll(d.stride(0)), ptr(order.contiguous()), ptr(seg_start),
                                          ptr(uniq.contiguous()), c_ll(n_seg), ptr(g), c_ll(g.stride(0)),
                                          c_int(1 if g.dtype == torch.float32 else 0), c_int(d.shape[1]), stream()),
          "embedding_grad")
    return True

