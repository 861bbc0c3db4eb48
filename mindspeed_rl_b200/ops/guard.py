"""Canary pads around kernel outputs (debug aid, off by default).

The kernels of this package write through raw pointers; an index error in one of them lands in whatever
the allocator placed next to the output.  With ``MSRL_DEBUG_CANARY=1`` every output tensor that an op
allocates on a CUDA device through :func:`empty` / :func:`empty_like` gets ``PAD`` bytes of a known
pattern in front of and behind it, and :func:`check` (called at worker stage boundaries and after every
GPU test) verifies that the pads of the tensors still alive are intact, naming the op that allocated a
damaged one.  This stands in for a memory checker where none can be run; it costs two small fills per
allocation and one comparison per live tensor at each check, so it stays off in production runs.
"""
from __future__ import annotations

import os
import traceback
import weakref
from typing import List, Tuple

import torch

PAD = 256
_PATTERN = 0xA5
_live: List[Tuple[weakref.ref, torch.Tensor, torch.Tensor, str]] = []


def enabled() -> bool:
    return os.environ.get("MSRL_DEBUG_CANARY", "0") == "1"


def _site() -> str:
    for fr in reversed(traceback.extract_stack(limit=6)[:-2]):
        if not fr.filename.endswith("guard.py"):
            return f"{os.path.basename(fr.filename)}:{fr.lineno} ({fr.name})"
    return "?"


def empty(*size, dtype=None, device=None, **kw) -> torch.Tensor:
    """``torch.empty`` with canary pads when the debug mode is on and the tensor lives on a CUDA device."""
    if not enabled() or kw.get("pin_memory") or torch.device(device if device is not None else "cpu").type != "cuda":
        return torch.empty(*size, dtype=dtype, device=device, **kw)
    shape = tuple(size[0]) if len(size) == 1 and isinstance(size[0], (tuple, list, torch.Size)) else tuple(size)
    dtype = dtype or torch.get_default_dtype()
    n = 1
    for d in shape:
        n *= int(d)
    nbytes = n * torch.empty(0, dtype=dtype).element_size()
    body = (nbytes + PAD - 1) // PAD * PAD                    # the tail pad starts on a PAD boundary
    raw = torch.empty(PAD + body + PAD, dtype=torch.uint8, device=device)
    front, back = raw[:PAD], raw[PAD + nbytes:]
    front.fill_(_PATTERN)
    back.fill_(_PATTERN)
    out = raw[PAD:PAD + nbytes].view(dtype).view(shape)
    _live.append((weakref.ref(out), front, back, _site()))
    return out


def empty_like(t: torch.Tensor, dtype=None, **kw) -> torch.Tensor:
    if not enabled() or not t.is_cuda:
        return torch.empty_like(t, dtype=dtype, **kw)
    return empty(t.shape, dtype=dtype or t.dtype, device=t.device)


def check(where: str = "") -> int:
    """Verify the pads of all guarded tensors that are still alive; forget the dead ones.  Returns the
    number of tensors checked; raises ``RuntimeError`` naming the allocation site of a damaged pad."""
    global _live
    if not _live:
        return 0
    torch.cuda.synchronize()
    keep, bad = [], []
    for ref, front, back, site in _live:
        if bool((front != _PATTERN).any()) or bool((back != _PATTERN).any()):
            side = "before" if bool((front != _PATTERN).any()) else "after"
            bad.append(f"{site}: bytes {side} the tensor were overwritten")
        elif ref() is not None:
            keep.append((ref, front, back, site))
    checked = len(_live)
    _live = keep
    if bad:
        raise RuntimeError(f"kernel wrote outside its output ({where}): " + "; ".join(bad))
    return checked
