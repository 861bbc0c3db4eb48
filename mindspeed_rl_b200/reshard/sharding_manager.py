"""Memory / weight choreography between the three phases of a co-located actor.

Modes (reference state machine: ``mindspeed_rl/workers/resharding/megatron_sharding_manager.py:113-218``):

* **infer**   -- rollout weights are produced from the training weights (zero-copy alias when
  the layouts coincide, otherwise the reshard plan executed by the reshard kernel), optional
  offload of optimizer state / gradient buffers / training weights to pinned host memory,
  weights bound into the rollout engine, KV cache allocated;
* **forward** -- training weights resident (log-prob passes);
* **train**   -- weights + gradient buffers + optimizer state resident.

Every transition reports its wall time so the trainer can log ``timing/resharding_to_infer``
(enter + exit infer) and ``timing/resharding_to_train``.
"""
from __future__ import annotations

import time
from typing import Callable, List, Optional

import torch

from ..parallel.ddp import DistributedDataParallel
from .alias import alias_rollout_weights


class GradBufferOffloader:
    """Release / re-create the flat gradient buffers (they hold no state between steps).  A buffer that
    is a slice of the job-wide peer-mapped arena stays resident; one with a peer-mapped segment of its
    own (``DistributedDataParallel(releasable_grads=True)``) or a plain allocation is really freed."""

    def __init__(self, ddp: Optional[DistributedDataParallel]):
        self.ddp = ddp
        self.released = False

    def release(self) -> None:
        if self.ddp is None or self.released:
            return
        for b in self.ddp.buffers:
            b.release_grads()
        self.released = True

    def restore(self) -> None:
        if self.ddp is None or not self.released:
            return
        for b in self.ddp.buffers:
            b.restore_grads()
        self.released = False


class ParamOffloader:
    """Swap the flat parameter buffers between the device and pinned host twins (same rule: a slice of
    the job-wide arena stays where it is)."""

    def __init__(self, ddp: Optional[DistributedDataParallel]):
        self.ddp = ddp
        self.host: List[Optional[torch.Tensor]] = []
        self.offloaded = False

    def offload(self) -> None:
        if self.ddp is None or self.offloaded:
            return
        if not self.host:
            self.host = [torch.empty(b.numel, dtype=b.param_dtype, pin_memory=b.device.type == "cuda")
                         for b in self.ddp.buffers]
        for b, h in zip(self.ddp.buffers, self.host):
            b.release_params(h)
        self.offloaded = True

    def onload(self) -> None:
        if self.ddp is None or not self.offloaded:
            return
        for b, h in zip(self.ddp.buffers, self.host):
            b.restore_params(h)
        self.offloaded = False


class ShardingManager:
    def __init__(self, train_model, rollout_engine, optimizer=None, *,
                 offload_train_optimizer: bool = False, offload_train_grad: bool = False,
                 offload_train_param: bool = False, num_kv_blocks: Optional[int] = None,
                 gpu_memory_utilization: float = 0.5, resharder=None,
                 build_weights: Optional[Callable] = None, headroom_bytes: int = 2 << 30):
        self.train_model = train_model
        self.core = train_model.module if hasattr(train_model, "module") else train_model
        self.engine = rollout_engine
        self.optimizer = optimizer
        self.offload_train_optimizer = offload_train_optimizer
        self.offload_train_grad = offload_train_grad
        self.offload_train_param = offload_train_param
        self.num_kv_blocks = num_kv_blocks
        self.gpu_memory_utilization = gpu_memory_utilization
        self.headroom_bytes = int(headroom_bytes)     # left free beside the KV cache for the forward's temporaries
        self.resharder = resharder           # reshard.planner.Resharder when layouts differ
        self.build_weights = build_weights
        ddp = train_model if isinstance(train_model, DistributedDataParallel) else None
        self.grad_offloader = GradBufferOffloader(ddp)
        self.param_offloader = ParamOffloader(ddp)
        self.mode = "train"
        self.last_timing = {}

    # ------------------------------------------------------------------------------------------
    def _kv_block_cap(self) -> Optional[int]:
        """Blocks that ``max_num_seqs`` sequences of ``max_model_len`` tokens can occupy at once (plus one
        block of slack each); ``None`` when extra blocks are useful as a prefix cache."""
        e = self.engine
        if getattr(e, "enable_prefix_caching", False):
            return None
        per_seq = (e.max_model_len + e.block_size - 1) // e.block_size + 1
        return max(int(e.max_num_seqs) * per_seq, 16)

    def _kv_budget(self) -> int:
        """Bytes the KV cache may take right now: free memory minus the forward's head-room, at most the
        configured fraction of the device."""
        free, total = torch.cuda.mem_get_info(self.engine.device)
        return min(free - self.headroom_bytes, int(total * self.gpu_memory_utilization))

    def _release_needed(self) -> bool:
        """Whether the training buffers marked for offload really have to go for the rollout: not when
        the KV cache reaches its useful size (``_kv_block_cap``) without them.  Freeing and re-creating
        peer-mapped segments is collective and costs a second per step on eight ranks, so the ranks of
        the team agree (all must answer the same) and skip it when none of them needs the memory."""
        if self.engine.device.type != "cuda" or self.num_kv_blocks:
            return True
        cap = self._kv_block_cap()
        if cap is None:
            return True
        enough = self._kv_budget() >= cap * self.engine.kv_bytes_per_block()
        import torch.distributed as dist

        ddp = self.grad_offloader.ddp
        owners = [b for b in (ddp.buffers if ddp is not None else []) if any(getattr(b, "_own", {}).values())]
        if owners and dist.is_initialized():
            # buffers with peer-mapped segments: the segment's team decides together (its group, or the
            # whole job when the arena spans it); plain allocations are released rank by rank
            t = torch.tensor([1 if enough else 0], dtype=torch.int32, device=self.engine.device)
            dist.all_reduce(t, op=dist.ReduceOp.MIN, group=owners[0]._team)
            enough = bool(int(t.item()))
        return not enough

    def _kv_blocks(self) -> int:
        if self.num_kv_blocks:
            return self.num_kv_blocks
        dev = self.engine.device
        if dev.type != "cuda":
            return 256
        blocks = max(int(self._kv_budget() // self.engine.kv_bytes_per_block()), 16)
        cap = self._kv_block_cap()
        if cap is not None:
            blocks = min(blocks, cap)          # more than every sequence at full length can use is only allocation time
        comm = getattr(self.engine, "comm", None)
        if comm is not None and comm.world_size > 1 and comm.group is not None:
            # the ranks of a rollout TP group run identical schedulers: they must agree on the cache
            # size (free memory differs a little from GPU to GPU), so all take the smallest
            import torch.distributed as dist

            t = torch.tensor([blocks], dtype=torch.int64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MIN, group=comm.group)
            blocks = int(t.item())
        return blocks

    def enter_infer_mode(self) -> float:
        t0 = time.time()
        if self.offload_train_optimizer and self.optimizer is not None:
            self.optimizer.offload_state()
        release = (self.offload_train_grad or (self.offload_train_param and self.resharder is not None)) \
            and self._release_needed()
        if self.offload_train_grad and release:
            self.grad_offloader.release()
        if self.resharder is not None:
            weights = self.resharder.reshard(self.core)
            if self.offload_train_param and release:
                self.param_offloader.offload()
        elif self.build_weights is not None:
            weights = self.build_weights(self.core)
        else:
            weights = alias_rollout_weights(self.core)
        self.engine.runner.bind_weights(weights)
        self._sync()
        t_kv = time.time()
        self.engine.init_cache(self._kv_blocks())
        self._sync()
        self.mode = "infer"
        dt = time.time() - t0
        self.last_timing["enter_infer"] = dt
        self.last_timing["kv_cache_alloc"] = time.time() - t_kv
        ms = self.resharder.device_ms() if self.resharder is not None else None
        self.last_timing["reshard_device"] = (ms or 0.0) / 1e3
        return dt

    def exit_infer_mode(self) -> float:
        t0 = time.time()
        self.engine.free_cache()
        if self.resharder is not None:
            self.engine.runner.bind_weights(None)
            self.resharder.release()
        self._sync()
        if self.engine.device.type == "cuda":
            torch.cuda.empty_cache()
        self.mode = "idle"
        dt = time.time() - t0
        self.last_timing["exit_infer"] = dt
        return dt

    def enter_forward_mode(self) -> None:
        self.param_offloader.onload()
        self.mode = "forward"

    def exit_forward_mode(self) -> None:
        self.mode = "idle"

    def enter_train_mode(self) -> float:
        t0 = time.time()
        self.param_offloader.onload()
        self.grad_offloader.restore()
        if self.optimizer is not None:
            self.optimizer.onload_state()
        self._sync()
        self.mode = "train"
        dt = time.time() - t0
        self.last_timing["enter_train"] = dt
        return dt

    def exit_train_mode(self) -> None:
        self.mode = "idle"

    def _sync(self) -> None:
        if self.engine.device.type == "cuda":
            torch.cuda.synchronize(self.engine.device)
