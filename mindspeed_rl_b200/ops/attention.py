"""Variable-length causal attention over packed token streams (training / prefill).

``attn_varlen_fwd(qkv, layout, cu_seqlens, max_seqlen)`` reads q/k/v heads straight out of
the fused QKV projection output (``QKVLayout``) and returns ``[T, nh*hd]`` plus the
log-sum-exp needed by ``attn_varlen_bwd``, which writes dq/dk/dv straight into a ``dqkv``
tensor of the same layout.  CUDA path: ``csrc/attention.cu``; CPU path: per-sequence fp32
softmax attention (also the test oracle).
"""
from __future__ import annotations

import ctypes
import math
import os
from typing import Optional, Tuple

import torch

from . import guard

from . import _lib
from ._lib import c_int, c_ll, check, ptr, stream
from .elementwise import _workspace
from .layouts import QKVLayout


def _layout_array(*specs) -> ctypes.Array:
    vals = []
    for _, (st, gs, hpg, hs) in specs:
        vals += [st, gs, hpg, hs]
    return (ctypes.c_longlong * len(vals))(*vals)


def _ref_attention(q, k, v, cu_q, cu_k, causal):
    """fp32 reference; q [Tq, nh, hd], k/v [Tk, nkv, hd]; returns out [Tq, nh, hd], lse [nh, Tq]."""
    tq, nh, hd = q.shape
    nkv = k.shape[1]
    rep = nh // nkv
    out = torch.zeros(tq, nh, hd, dtype=torch.float32, device=q.device)
    lse = torch.zeros(nh, tq, dtype=torch.float32, device=q.device)
    scale = 1.0 / math.sqrt(hd)
    cq, ck = cu_q.tolist(), cu_k.tolist()
    for b in range(len(cq) - 1):
        qs, qe, ks, ke = cq[b], cq[b + 1], ck[b], ck[b + 1]
        if qe == qs:
            continue
        qi = q[qs:qe].float().transpose(0, 1)                       # [nh, Lq, hd]
        ki = k[ks:ke].float().transpose(0, 1).repeat_interleave(rep, dim=0)
        vi = v[ks:ke].float().transpose(0, 1).repeat_interleave(rep, dim=0)
        s = torch.matmul(qi, ki.transpose(1, 2)) * scale            # [nh, Lq, Lk]
        if causal:
            lq, lk = qe - qs, ke - ks
            i = torch.arange(lq, device=q.device).unsqueeze(1)
            j = torch.arange(lk, device=q.device).unsqueeze(0)
            s = s.masked_fill(j > i + (lk - lq), float("-inf"))
        l = torch.logsumexp(s, dim=-1)
        p = torch.exp(s - l.unsqueeze(-1))
        out[qs:qe] = torch.matmul(p, vi).transpose(0, 1)
        lse[:, qs:qe] = l
    return out, lse


def use_tcgen05_attention() -> bool:
    """The tcgen05 forward kernel (``csrc/attention_tcgen05.cu``) serves head size 128 unless
    ``MSRL_ATTN_TCGEN05=0``; everything else runs the mma.sync kernel of ``csrc/attention.cu``."""
    return os.environ.get("MSRL_ATTN_TCGEN05", "1") != "0"


_NOT_SUPPORTED = 801   # cudaErrorNotSupported: the shape is outside the tcgen05 kernel's cover


def attn_varlen_fwd(qkv: torch.Tensor, layout: QKVLayout, cu_seqlens: torch.Tensor, max_seqlen: int,
                    causal: bool = True, kv: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                    cu_seqlens_k: Optional[torch.Tensor] = None
                    ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns ``(out [T, nh*hd], lse [nh, T] fp32)``.

    ``kv=(k, v)`` with contiguous ``[Tk, nkv, hd]`` tensors and ``cu_seqlens_k`` selects the
    prefix-attention form (queries from ``qkv``, keys/values from ``kv``; the causal mask is
    bottom-right aligned).
    """
    t = qkv.shape[0]
    nh, nkv, hd = layout.num_heads, layout.num_kv_heads, layout.head_dim
    batch = cu_seqlens.numel() - 1
    cu_k = cu_seqlens if cu_seqlens_k is None else cu_seqlens_k
    if _lib.use_kernels(qkv, cu_seqlens):
        flat = qkv.view(-1)
        qs = layout.q()
        if kv is None:
            ks, vs = layout.k(), layout.v()
            kb, vb = flat[ks[0]:], flat[vs[0]:]
        else:
            ks = vs = (0, (nkv * hd, 0, nkv, hd))
            kb, vb = kv[0].contiguous().view(-1), kv[1].contiguous().view(-1)
        lay = _layout_array(qs, ks, vs)
        out = guard.empty(t, nh * hd, device=qkv.device, dtype=qkv.dtype)
        lse = guard.empty(nh, t, device=qkv.device, dtype=torch.float32)
        if hd == 128 and use_tcgen05_attention():
            from .gemm import _status_word
            tk = t if kv is None else kv[0].shape[0]
            rc = _lib.load().msrl_flash_attn_varlen_fwd_tcgen05(
                ptr(flat[qs[0]:]), ptr(kb), ptr(vb), lay, ptr(out), c_ll(nh * hd), ptr(lse),
                ptr(cu_seqlens), ptr(cu_k), c_int(batch), c_int(int(max_seqlen)), c_int(nh), c_int(nkv),
                c_ll(t), c_ll(tk), c_int(hd), c_int(1 if causal else 0),
                ptr(_status_word(qkv.device)), stream())
            if rc != _NOT_SUPPORTED:
                check(rc, "flash_attn_varlen_fwd_tcgen05")
                return out, lse
        check(_lib.load().msrl_flash_attn_varlen_fwd(
            ptr(flat[qs[0]:]), ptr(kb), ptr(vb), lay, ptr(out), c_ll(nh * hd), ptr(lse),
            ptr(cu_seqlens), ptr(cu_k), c_int(batch), c_int(int(max_seqlen)), c_int(nh), c_int(nkv),
            c_ll(t), c_int(hd), c_int(1 if causal else 0), stream()), "flash_attn_varlen_fwd")
        return out, lse
    q, k, v = layout.split(qkv)
    if kv is not None:
        k, v = kv
    o, lse = _ref_attention(q, k, v, cu_seqlens, cu_k, causal)
    return o.reshape(t, nh * hd).to(qkv.dtype), lse


def attn_varlen_bwd(dout: torch.Tensor, qkv: torch.Tensor, out: torch.Tensor, lse: torch.Tensor,
                    layout: QKVLayout, cu_seqlens: torch.Tensor, max_seqlen: int,
                    causal: bool = True) -> torch.Tensor:
    """Returns ``dqkv`` with the layout of ``qkv`` (self-attention form only)."""
    t = qkv.shape[0]
    nh, nkv, hd = layout.num_heads, layout.num_kv_heads, layout.head_dim
    batch = cu_seqlens.numel() - 1
    if _lib.use_kernels(qkv, dout, out):
        flat = qkv.view(-1)
        dqkv = guard.empty_like(qkv)
        dflat = dqkv.view(-1)
        qs, ks, vs = layout.q(), layout.k(), layout.v()
        lay = _layout_array(qs, ks, vs)
        delta = _workspace("attn_delta", nh * t, qkv.device)
        do = dout.contiguous()
        if hd == 128 and use_tcgen05_attention():
            from .gemm import _status_word
            rc = _lib.load().msrl_flash_attn_varlen_bwd_tcgen05(
                ptr(flat[qs[0]:]), ptr(flat[ks[0]:]), ptr(flat[vs[0]:]), lay, ptr(out), ptr(do),
                c_ll(nh * hd), ptr(lse), ptr(delta), ptr(dflat[qs[0]:]), ptr(dflat[ks[0]:]),
                ptr(dflat[vs[0]:]), ptr(cu_seqlens), ptr(cu_seqlens), c_int(batch),
                c_int(int(max_seqlen)), c_int(int(max_seqlen)), c_int(nh), c_int(nkv), c_ll(t), c_ll(t),
                c_int(hd), c_int(1 if causal else 0), ptr(_status_word(qkv.device)), stream())
            if rc != _NOT_SUPPORTED:
                check(rc, "flash_attn_varlen_bwd_tcgen05")
                return dqkv
        check(_lib.load().msrl_flash_attn_varlen_bwd(
            ptr(flat[qs[0]:]), ptr(flat[ks[0]:]), ptr(flat[vs[0]:]), lay, ptr(out), ptr(do),
            c_ll(nh * hd), ptr(lse), ptr(delta), ptr(dflat[qs[0]:]), ptr(dflat[ks[0]:]),
            ptr(dflat[vs[0]:]), ptr(cu_seqlens), ptr(cu_seqlens), c_int(batch),
            c_int(int(max_seqlen)), c_int(int(max_seqlen)), c_int(nh), c_int(nkv), c_ll(t), c_int(hd),
            c_int(1 if causal else 0), stream()), "flash_attn_varlen_bwd")
        return dqkv
    # reference: autograd through the fp32 formulation
    with torch.enable_grad():
        x = qkv.detach().float().requires_grad_(True)
        q, k, v = layout.split(x)
        o, _ = _ref_attention(q, k, v, cu_seqlens, cu_seqlens, causal)
        (gx,) = torch.autograd.grad(o.reshape(t, nh * hd), x, dout.float())
    return gx.to(qkv.dtype)


def attn_kv_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_q: torch.Tensor, cu_k: torch.Tensor,
                max_q: int, causal: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    """Attention of contiguous ``q [Tq, nh, hd]`` over separate ``k, v [Tk, nkv, hd]`` (packed
    sequences, ``cu_q`` / ``cu_k``); returns ``(out [Tq, nh*hd], lse [nh, Tq])``.  The block of the
    ring algorithm of context parallelism."""
    tq, nh, hd = q.shape
    tk, nkv, _ = k.shape
    batch = cu_q.numel() - 1
    if _lib.use_kernels(q, k, v):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        out = guard.empty(tq, nh * hd, device=q.device, dtype=q.dtype)
        lse = guard.empty(nh, tq, device=q.device, dtype=torch.float32)
        lay = (ctypes.c_longlong * 12)(nh * hd, 0, nh, hd, nkv * hd, 0, nkv, hd, nkv * hd, 0, nkv, hd)
        if hd == 128 and use_tcgen05_attention():
            from .gemm import _status_word
            rc = _lib.load().msrl_flash_attn_varlen_fwd_tcgen05(
                ptr(q), ptr(k), ptr(v), lay, ptr(out), c_ll(nh * hd), ptr(lse), ptr(cu_q), ptr(cu_k), c_int(batch),
                c_int(int(max_q)), c_int(nh), c_int(nkv), c_ll(tq), c_ll(tk), c_int(hd), c_int(1 if causal else 0),
                ptr(_status_word(q.device)), stream())
            if rc != _NOT_SUPPORTED:
                check(rc, "flash_attn_varlen_fwd_tcgen05")
                return out, lse
        check(_lib.load().msrl_flash_attn_varlen_fwd(
            ptr(q), ptr(k), ptr(v), lay, ptr(out), c_ll(nh * hd), ptr(lse), ptr(cu_q), ptr(cu_k), c_int(batch),
            c_int(int(max_q)), c_int(nh), c_int(nkv), c_ll(tq), c_int(hd), c_int(1 if causal else 0), stream()),
            "flash_attn_varlen_fwd")
        return out, lse
    o, lse = _ref_attention(q, k, v, cu_q, cu_k, causal)
    return o.reshape(tq, nh * hd).to(q.dtype), lse


def attn_kv_bwd(dout: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor,
                lse: torch.Tensor, cu_q: torch.Tensor, cu_k: torch.Tensor, max_q: int, max_k: int, causal: bool
                ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Gradients of one (q block, kv block) pair given the output and log-sum-exp of the WHOLE
    attention row (``out``, ``lse``: what the forward produced after merging all blocks), which is
    what makes the per-block gradients add up.  Contiguous ``q [Tq, nh, hd]``, ``k, v [Tk, nkv, hd]``;
    returns ``(dq, dk, dv)`` of the same shapes."""
    tq, nh, hd = q.shape
    tk, nkv, _ = k.shape
    batch = cu_q.numel() - 1
    if _lib.use_kernels(q, k, v, dout):
        q, k, v, do = q.contiguous(), k.contiguous(), v.contiguous(), dout.contiguous()
        dq, dk, dv = guard.empty_like(q), guard.empty_like(k), guard.empty_like(v)
        delta = _workspace("attn_delta", nh * tq, q.device)
        # contiguous [T, heads, hd]: head h starts at column h * hd
        lay = (ctypes.c_longlong * 12)(nh * hd, 0, nh, hd, nkv * hd, 0, nkv, hd, nkv * hd, 0, nkv, hd)
        if hd == 128 and use_tcgen05_attention():
            from .gemm import _status_word
            rc = _lib.load().msrl_flash_attn_varlen_bwd_tcgen05(
                ptr(q), ptr(k), ptr(v), lay, ptr(out), ptr(do), c_ll(nh * hd), ptr(lse), ptr(delta), ptr(dq),
                ptr(dk), ptr(dv), ptr(cu_q), ptr(cu_k), c_int(batch), c_int(int(max_q)), c_int(int(max_k)),
                c_int(nh), c_int(nkv), c_ll(tq), c_ll(tk), c_int(hd), c_int(1 if causal else 0),
                ptr(_status_word(q.device)), stream())
            if rc != _NOT_SUPPORTED:
                check(rc, "flash_attn_varlen_bwd_tcgen05")
                return dq, dk, dv
        check(_lib.load().msrl_flash_attn_varlen_bwd(
            ptr(q), ptr(k), ptr(v), lay, ptr(out), ptr(do), c_ll(nh * hd), ptr(lse), ptr(delta), ptr(dq), ptr(dk),
            ptr(dv), ptr(cu_q), ptr(cu_k), c_int(batch), c_int(int(max_q)), c_int(int(max_k)), c_int(nh),
            c_int(nkv), c_ll(tq), c_int(hd), c_int(1 if causal else 0), stream()), "flash_attn_varlen_bwd")
        return dq, dk, dv
    # reference: P from the given lse, then the usual formulas (fp32)
    rep = nh // nkv
    scale = 1.0 / math.sqrt(hd)
    dq, dk, dv = torch.zeros_like(q, dtype=torch.float32), torch.zeros_like(k, dtype=torch.float32), \
        torch.zeros_like(v, dtype=torch.float32)
    of, dof = out.float().view(tq, nh, hd), dout.float().view(tq, nh, hd)
    delta = (of * dof).sum(-1)                                              # [Tq, nh]
    cq, ck = cu_q.tolist(), cu_k.tolist()
    for b in range(batch):
        qs, qe, ks, ke = cq[b], cq[b + 1], ck[b], ck[b + 1]
        if qe == qs or ke == ks:
            continue
        qi = q[qs:qe].float().transpose(0, 1)                                # [nh, Lq, hd]
        ki = k[ks:ke].float().transpose(0, 1).repeat_interleave(rep, dim=0)
        vi = v[ks:ke].float().transpose(0, 1).repeat_interleave(rep, dim=0)
        s = torch.matmul(qi, ki.transpose(1, 2)) * scale
        if causal:
            lq, lk = qe - qs, ke - ks
            i = torch.arange(lq).unsqueeze(1)
            j = torch.arange(lk).unsqueeze(0)
            s = s.masked_fill(j > i + (lk - lq), float("-inf"))
        p = torch.exp(s - lse[:, qs:qe].unsqueeze(-1))
        doi = dof[qs:qe].transpose(0, 1)
        dvi = torch.matmul(p.transpose(1, 2), doi)
        dp = torch.matmul(doi, vi.transpose(1, 2))
        ds = p * (dp - delta[qs:qe].t().unsqueeze(-1)) * scale
        dq[qs:qe] = torch.matmul(ds, ki).transpose(0, 1)
        dki = torch.matmul(ds.transpose(1, 2), qi)
        dk[ks:ke] = dki.view(nkv, rep, ke - ks, hd).sum(1).transpose(0, 1)
        dv[ks:ke] = dvi.view(nkv, rep, ke - ks, hd).sum(1).transpose(0, 1)
    return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype)


def attn_merge_(acc_o: torch.Tensor, acc_l: torch.Tensor, o: torch.Tensor, l: torch.Tensor,
                rows: Optional[torch.Tensor] = None) -> None:
    """Fold a block result into the running result of an attention over disjoint key sets, in place:
    ``acc_o [T, nh, hd]`` fp32 and ``acc_l [nh, T]`` (log-sum-exp) absorb ``o [Tb, nh*hd]`` /
    ``l [nh, Tb]``; ``rows`` (int64 ``[Tb]``) names the running rows the block rows belong to."""
    t, nh, hd = acc_o.shape
    tb = o.shape[0]
    if _lib.use_kernels(acc_o, acc_l, o, l) and o.dtype == torch.bfloat16 and acc_o.is_contiguous() \
            and acc_l.is_contiguous() and hd % 8 == 0:
        check(_lib.load().msrl_attn_merge(ptr(acc_o), ptr(acc_l), c_ll(t), ptr(o.contiguous()), ptr(l.contiguous()),
                                          c_ll(tb), ptr(rows), c_int(nh), c_int(hd), stream()), "attn_merge")
        return
    ob = o.float().view(tb, nh, hd)
    if rows is None:
        lt = torch.logaddexp(acc_l, l)
        wa, wb = torch.exp(acc_l - lt), torch.exp(l - lt)
        acc_o.mul_(torch.nan_to_num(wa).t().unsqueeze(-1)).add_(ob * torch.nan_to_num(wb).t().unsqueeze(-1))
        acc_l.copy_(lt)
    else:
        al = acc_l[:, rows]
        lt = torch.logaddexp(al, l)
        wa, wb = torch.nan_to_num(torch.exp(al - lt)), torch.nan_to_num(torch.exp(l - lt))
        acc_o[rows] = acc_o[rows] * wa.t().unsqueeze(-1) + ob * wb.t().unsqueeze(-1)
        acc_l[:, rows] = lt
