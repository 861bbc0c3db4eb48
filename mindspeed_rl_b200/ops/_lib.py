"""Loader of the in-tree CUDA kernel library (``_C/libmsrl_b200.so``).

Policy: on a machine with a GPU the library *must* be present -- every op raises if it is
missing rather than silently running an eager PyTorch path.  Without a GPU (CPU-only
development, gloo tests) the ops run their PyTorch reference implementation.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path
from typing import Optional

import torch

_LIB_PATH = Path(__file__).resolve().parent.parent / "_C" / "libmsrl_b200.so"
_lib: Optional[ctypes.CDLL] = None
_launches = 0


class KernelLibraryMissing(RuntimeError):
    pass


def lib_path() -> Path:
    return _LIB_PATH


def load() -> ctypes.CDLL:
    """Return the kernel library, building it first when ``MSRL_AUTO_BUILD=1``."""
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists() and os.environ.get("MSRL_AUTO_BUILD", "0") == "1":
        from ..csrc import build as _build

        _build.build()
    if not _LIB_PATH.exists():
        raise KernelLibraryMissing(
            f"{_LIB_PATH} not found. Build it with `python -m mindspeed_rl_b200.csrc.build` "
            f"(or `python -c 'import __graft_entry__ as g; g.build()'`).")
    _lib = ctypes.CDLL(str(_LIB_PATH))
    return _lib


def available() -> bool:
    return _LIB_PATH.exists()


def use_kernels(*tensors: torch.Tensor) -> bool:
    """True when the CUDA kernels must be used for these tensors (all on a CUDA device)."""
    if not tensors or not all(t.is_cuda for t in tensors if t is not None):
        return False
    load()  # raises loudly on a GPU box without the library
    return True


def ptr(t: Optional[torch.Tensor]) -> Optional[ctypes.c_void_p]:
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def check(code: int, what: str) -> None:
    global _launches
    _launches += 1
    if code != 0:
        raise RuntimeError(f"kernel launch '{what}' failed with CUDA error code {code}")


def launch_count() -> int:
    """Number of kernel-library entry-point calls made by this process (bench bookkeeping)."""
    return _launches


def reset_launch_count() -> None:
    global _launches
    _launches = 0


c_int = ctypes.c_int
c_ll = ctypes.c_longlong
c_ull = ctypes.c_ulonglong
c_float = ctypes.c_float
