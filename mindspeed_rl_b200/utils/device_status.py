"""Host-side read of the status words that the kernels' bounded waits report through."""
from __future__ import annotations


def check_device_status(stage: str = "") -> None:
    """Stage boundary: read the status words the kernels' bounded waits report through (tcgen05
    pipelines, peer-memory barriers and slabs) and raise if one of them gave up, instead of handing
    a silently incomplete result to the next stage.  One small device-to-host read per stage; no-op
    when no such kernel ran in this process."""
    from ..ops import gemm
    from ..parallel.symm import get_arena
    for dev in list(gemm._status):
        gemm.check_status(dev, f"stage {stage}: tcgen05 kernel")
    arena = get_arena()
    if arena is not None:
        arena.check()
    from ..ops import guard
    if guard.enabled():
        guard.check(f"stage {stage}")      # debug mode: canary pads around the kernels' outputs
