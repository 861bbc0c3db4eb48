"""Front-end of the tcgen05 / TMA GEMM (``csrc/gemm_tcgen05.cu``).

``gemm_bf16_tn(a, b)`` computes ``a @ b.T`` for row-major bf16 ``a [M, K]`` and ``b [N, K]`` (the
``x @ W.T`` of every linear layer) on the 5th-generation tensor cores, and
``lmhead_stats(h, w, labels, ...)`` runs the LM head with the log-softmax statistics fused into
the epilogue so that logits never reach HBM.  Both kernels report a status word: a non-zero
value means one of their bounded waits expired and the result must be discarded.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

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
        out = torch.empty(m, n, device=a.device, dtype=torch.bfloat16)
    check(_lib.load().msrl_gemm_bf16_tn(ptr(a), c_ll(a.stride(0)), ptr(b), c_ll(b.stride(0)), ptr(out),
                                        c_ll(out.stride(0)), c_int(m), c_int(n), c_int(k),
                                        ptr(_status_word(a.device)), stream()), "gemm_bf16_tn")
    return out


def lmhead_stats(h: torch.Tensor, w: torch.Tensor, labels: torch.Tensor, inv_temp: float,
                 vocab_offset: int = 0) -> Tuple[torch.Tensor, int]:
    """Per-row, per-256-column-tile softmax statistics of ``(h @ w.T) * inv_temp``.

    Returns ``(stats [tiles, M, 4] fp32, tiles)``; feed them to ``msrl_logprob_finish``.
    """
    m, k = h.shape
    n = w.shape[0]
    L = _lib.load()
    tiles = L.msrl_lmhead_stats_tiles(c_int(n))
    stats = torch.empty(tiles, m, 4, device=h.device, dtype=torch.float32)
    check(L.msrl_lmhead_stats(ptr(h), c_ll(h.stride(0)), ptr(w), c_ll(w.stride(0)), ptr(labels),
                              c_int(vocab_offset), c_float(inv_temp), ptr(stats), c_int(m), c_int(n),
                              c_int(k), ptr(_status_word(h.device)), stream()), "lmhead_stats")
    return stats, tiles


def tcgen05_usable(*tensors: torch.Tensor) -> bool:
    return all(_ok_operand(t) for t in tensors) and _lib.available()
