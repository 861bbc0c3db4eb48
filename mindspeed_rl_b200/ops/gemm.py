"""Front-end of the tcgen05 / TMA GEMM (``csrc/gemm_tcgen05.cu``).

``gemm_bf16_tn(a, b)`` computes ``a @ b.T`` for row-major bf16 ``a [M, K]`` and ``b [N, K]`` (the
``x @ W.T`` of every linear layer) on the 5th-generation tensor cores, and
``lmhead_stats(h, w, labels, ...)`` runs the LM head with the log-softmax statistics fused into
the epilogue so that logits never reach HBM.  Both kernels report a status word: a non-zero
value means one of their bounded waits expired and the result must be discarded.
"""
from __future__ import annotations

import os
from typing import Optional, Tuple

import torch

from . import guard

from . import _lib
from ._lib import c_float, c_int, c_ll, check, ptr, stream


class KernelTimeout(RuntimeError):
    """A bounded wait inside a kernel expired (pipeline stalled); the output is invalid."""


_status = {}


def _status_word(device) -> torch.Tensor:
    t = _status.get(device)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _status[device] = t
    return t


def check_status(device, what: str = "tcgen05 gemm") -> None:
    """Synchronising check of the status word (call at phase boundaries, not per launch)."""
    t = _status.get(torch.device(device))
    if t is not None and int(t.item()) != 0:
        code = int(t.item())
        t.zero_()
        raise KernelTimeout(f"{what}: device-side wait timed out (code {code})")


def _ok_operand(t: torch.Tensor) -> bool:
    return (t.is_cuda and t.dtype == torch.bfloat16 and t.dim() == 2 and t.stride(1) == 1
            and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0 and t.shape[1] % 8 == 0)


def gemm_bf16_tn(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a [M, K] @ b [N, K].T -> [M, N]`` (bf16)."""
    if not (_ok_operand(a) and _ok_operand(b)) or not _lib.use_kernels(a, b):
        r = torch.matmul(a, b.t())
        if out is not None:
            out.copy_(r)
            return out
        return r
    m, k = a.shape
    n = b.shape[0]
    if out is None:
        out = guard.empty(m, n, device=a.device, dtype=torch.bfloat16)
    check(_lib.load().msrl_gemm_bf16_tn(ptr(a), c_ll(a.stride(0)), ptr(b), c_ll(b.stride(0)), ptr(out),
                                        c_ll(out.stride(0)), c_int(m), c_int(n), c_int(k),
                                        ptr(_status_word(a.device)), stream()), "gemm_bf16_tn")
    return out


_OUT_MODES = {"store": 0, "acc_f32": 1, "acc_bf16": 2}


def _ok_matrix(t: torch.Tensor) -> bool:
    return (t.is_cuda and t.dtype == torch.bfloat16 and t.dim() == 2 and t.stride(1) == 1
            and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0)


def pair_usable(*tensors: torch.Tensor) -> bool:
    """True when the CTA-pair GEMM can take these bf16 matrices as operands (CUDA, contiguous rows,
    16-byte aligned, leading dimensions and row lengths multiples of 8)."""
    return all(_ok_matrix(t) and t.shape[1] % 8 == 0 for t in tensors) and _lib.available()


def gemm_pair(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
              out: Optional[torch.Tensor] = None, mode: str = "store",
              bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Dense GEMM on CTA pairs (``csrc/gemm2cta_tcgen05.cu``): ``C[M, N] (+)= op(a) @ op(b).T``.

    ``a`` is ``[M, K]`` (``a_mn=False``) or stored transposed ``[K, M]`` (``a_mn=True``); ``b`` is
    ``[N, K]`` or stored transposed ``[K, N]``.  ``mode``: ``store`` (bf16 result, optional bias
    ``[N]``), ``acc_f32`` / ``acc_bf16`` (add into an existing fp32 / bf16 ``out``)."""
    m, k = (a.shape[1], a.shape[0]) if a_mn else a.shape
    n = b.shape[1] if b_mn else b.shape[0]
    if (b.shape[0] if b_mn else b.shape[1]) != k:
        raise ValueError("inner dimensions do not match")
    if out is None:
        if mode != "store":
            raise ValueError("accumulating modes need an output tensor")
        out = guard.empty(m, n, device=a.device, dtype=torch.bfloat16)
    check(_lib.load().msrl_gemm_pair_bf16(
        ptr(a), c_ll(a.stride(0)), c_int(int(a_mn)), ptr(b), c_ll(b.stride(0)), c_int(int(b_mn)), ptr(out),
        c_ll(out.stride(0)), c_int(_OUT_MODES[mode]), ptr(bias), c_int(m), c_int(n), c_int(k),
        ptr(_status_word(a.device)), stream()), "gemm_pair_bf16")
    return out


def pair_enabled() -> bool:
    """``MSRL_PAIR_GEMM=0`` sends the dense linears to the library GEMM (comparison runs)."""
    return os.environ.get("MSRL_PAIR_GEMM", "1") == "1"


def _pair_pays(m: int, n: int) -> bool:
    """The pair kernel works on 256 x 256 output tiles, one pair of SMs each: below a few dozen
    tiles (decode-sized problems) most of the machine would idle, so those go to the library."""
    return pair_enabled() and m > 128 and ((m + 255) // 256) * ((n + 255) // 256) >= 48


def gemm_pair_splitk(x: torch.Tensor, w: torch.Tensor, splits: int, bias: Optional[torch.Tensor] = None,
                     out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x [M, K] @ w [N, K].T (+ bias)`` for small ``M`` (decode steps) on the CTA-pair kernel with the
    reduction cut into ``splits`` pieces: tiles x pieces fills the machine although ``M x N`` alone is a
    handful of tiles, each piece streams its part of the weight once, and a second kernel adds the
    fp32 partial tiles in a fixed order."""
    m, k = x.shape
    n = w.shape[0]
    if out is None:
        out = guard.empty(m, n, device=x.device, dtype=torch.bfloat16)
    part = guard.empty(splits * m * n, device=x.device, dtype=torch.float32)
    check(_lib.load().msrl_gemm_pair_splitk_bf16(
        ptr(x), c_ll(x.stride(0)), ptr(w), c_ll(w.stride(0)), ptr(part), ptr(out), c_ll(out.stride(0)), ptr(bias),
        c_int(m), c_int(n), c_int(k), c_int(splits), ptr(_status_word(x.device)), stream()), "gemm_pair_splitk_bf16")
    return out


def splitk_plan(m: int, n: int, k: int) -> int:
    """Pieces to cut the reduction of a small-``M`` GEMM into (0: do not split)."""
    if not pair_enabled() or os.environ.get("MSRL_SPLITK_GEMM", "1") != "1":
        return 0
    return int(_lib.load().msrl_gemm_pair_splitk_plan(c_int(m), c_int(n), c_int(k)))


def linear_fwd(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x [T, K] @ w [N, K].T (+ bias)``: the forward of every dense linear."""
    if (x.is_cuda and pair_usable(x, w) and _lib.use_kernels(x, w)
            and (bias is None or (bias.dtype == torch.bfloat16 and bias.data_ptr() % 16 == 0))):
        m, n, k = x.shape[0], w.shape[0], x.shape[1]
        if _pair_pays(m, n):
            return gemm_pair(x, w, bias=bias)
        if 128 < m <= 256:
            splits = splitk_plan(m, n, k)
            if splits >= 2:
                return gemm_pair_splitk(x, w, splits, bias=bias)
    if bias is not None:
        return torch.addmm(bias, x, w.t())
    return torch.matmul(x, w.t())


def linear_dgrad(dy: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``dy [T, N] @ w [N, K]``: input gradient of a linear, reading ``w`` where it is."""
    if dy.is_cuda and _pair_pays(dy.shape[0], w.shape[1]) and pair_usable(dy, w) and _lib.use_kernels(dy, w):
        return gemm_pair(dy, w, b_mn=True)
    return torch.matmul(dy, w)


def linear_wgrad_(grad: torch.Tensor, dy: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """``grad [N, K] += dy [T, N].T @ x [T, K]`` in place (``grad`` bf16 or fp32)."""
    if (dy.is_cuda and _pair_pays(dy.shape[1], x.shape[1]) and pair_usable(dy, x) and _lib.use_kernels(dy, x, grad)
            and grad.dim() == 2 and grad.stride(1) == 1 and dy.shape[0] % 8 == 0 and grad.stride(0) % 8 == 0
            and grad.dtype in (torch.float32, torch.bfloat16) and grad.data_ptr() % 16 == 0):
        gemm_pair(dy, x, a_mn=True, b_mn=True, out=grad,
                  mode="acc_f32" if grad.dtype == torch.float32 else "acc_bf16")
        return grad
    if grad.dtype == dy.dtype:
        return grad.addmm_(dy.t(), x)
    return grad.add_(torch.matmul(dy.t(), x))


def lmhead_stats(h: torch.Tensor, w: torch.Tensor, labels: torch.Tensor, inv_temp: float,
                 vocab_offset: int = 0) -> Tuple[torch.Tensor, int]:
    """Per-row, per-256-column-tile softmax statistics of ``(h @ w.T) * inv_temp``.

    Returns ``(stats [tiles, M, 4] fp32, tiles)``; feed them to ``msrl_logprob_finish``.
    """
    m, k = h.shape
    n = w.shape[0]
    L = _lib.load()
    tiles = L.msrl_lmhead_stats_tiles(c_int(n))
    stats = guard.empty(tiles, m, 4, device=h.device, dtype=torch.float32)
    check(L.msrl_lmhead_stats(ptr(h), c_ll(h.stride(0)), ptr(w), c_ll(w.stride(0)), ptr(labels),
                              c_int(vocab_offset), c_float(inv_temp), ptr(stats), c_int(m), c_int(n),
                              c_int(k), ptr(_status_word(h.device)), stream()), "lmhead_stats")
    return stats, tiles


def tcgen05_usable(*tensors: torch.Tensor) -> bool:
    return all(_ok_operand(t) for t in tensors) and _lib.available()
