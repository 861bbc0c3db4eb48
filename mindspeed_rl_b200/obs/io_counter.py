"""Host<->device traffic accounting and pinned staging for step inputs.

``to_device`` is the one place where per-step host data (token ids, positions, slot tables,
training batches) enters the GPU: it goes through a pinned staging tensor and an async copy, and
the bytes are counted so that benchmarks can report ``h2d_bytes_per_step``.  ``to_host`` is the
counted counterpart for results read back (sampled tokens, losses, log-probs).
"""
from __future__ import annotations

from typing import Any

import numpy as np
import torch

_h2d = 0
_d2h = 0


def reset() -> None:
    global _h2d, _d2h
    _h2d = _d2h = 0


def counters():
    return _h2d, _d2h


def to_device(data: Any, dtype: torch.dtype, device) -> torch.Tensor:
    """Host list / ndarray / CPU tensor -> device tensor through pinned memory."""
    global _h2d
    device = torch.device(device)
    if torch.is_tensor(data):
        host = data.to(dtype)
    elif isinstance(data, np.ndarray):
        host = torch.from_numpy(data).to(dtype)
    else:
        host = torch.tensor(data, dtype=dtype)
    if device.type != "cuda":
        return host.to(device)
    _h2d += host.numel() * host.element_size()
    return host.pin_memory().to(device, non_blocking=True)


def count_d2h(nbytes: int) -> None:
    """Account for a device->host copy issued by the caller itself (an asynchronous pinned read)."""
    global _d2h
    _d2h += int(nbytes)


def to_host(t: torch.Tensor) -> torch.Tensor:
    global _d2h
    if t.is_cuda:
        _d2h += t.numel() * t.element_size()
    return t.cpu()
