"""Worker groups: the handle a trainer uses to drive all ranks of one role.

The trainer-facing API is the one of the reference's ``RayActorGroup``
(``mindspeed_rl/workers/scheduler/launcher.py:125-352``): ``initialize``, stage methods with a
``blocking`` flag, ``wait_all_ref_objs_run_over``, ``sync_init_transfer_dock``,
``save_checkpoint``, ``get_iteration``.

``SPMDWorkerGroup`` is the native B200 deployment: one process per GPU launched by
``torchrun``; every process runs the same trainer loop.  A group owns a set of global ranks
(``runtime.placement``); a stage call is a plain local call on the member ranks (the
collectives inside keep them in lock-step) and returns at once on every other rank.  Rank 0
is the *driver*: it owns the experience store (served to the other ranks over
``runtime.rpc``) and runs the CPU stages (rule reward, advantages, metrics, logging).

``blocking`` keeps the meaning it has for the trainers: a blocking stage is finished on all of
its ranks before any rank starts the next stage (a barrier over the job when roles live on
disjoint ranks); a non-blocking stage lets the other roles' ranks run ahead, so e.g. the
reference forward on its GPUs overlaps the actor's old-log-prob pass, until
``wait_all_ref_objs_run_over`` joins them.  When all roles share the same ranks the stages of one
process run one after the other anyway and no extra synchronisation is added.
"""
from __future__ import annotations

import os
from typing import Any, Callable, List, Optional, Sequence

import torch
import torch.distributed as dist


class SPMDWorkerGroup:
    def __init__(self, worker=None, num_gpus: Optional[int] = None, *, ranks: Optional[Sequence[int]] = None,
                 factory: Optional[Callable[[], Any]] = None, overlapping: bool = False):
        """``worker``: the local worker object (co-located groups: every rank is a member), or
        ``factory`` + ``ranks``: the worker is built only on the member ranks.  ``overlapping``
        says that some other group of the job lives on different ranks, i.e. that ``blocking``
        has something to order."""
        inited = dist.is_available() and dist.is_initialized()
        self.rank = dist.get_rank() if inited else 0
        self.world_size = dist.get_world_size() if inited else 1
        self.ranks = list(ranks) if ranks is not None else list(range(self.world_size))
        self.is_member = self.rank in self.ranks
        self.overlapping = bool(overlapping) and self.world_size > 1
        if worker is None and factory is not None and self.is_member:
            worker = factory()
        self.worker = worker if self.is_member else None
        self.num_npus = num_gpus or len(self.ranks)
        self.rl_config = getattr(worker, "rl_config", None)
        self.megatron_config = getattr(worker, "actor_config", getattr(worker, "megatron_config", None))
        self.initialized = False
        self._pending = 0

    @property
    def is_driver(self) -> bool:
        return self.rank == 0

    def initialize(self):
        if self.worker is not None:
            self.worker.initialize()
        self.initialized = True
        return self

    def sync_init_transfer_dock(self, td, mm_td=None, sampling_transfer_dock=None) -> None:
        if self.worker is not None:
            self.worker.init_transfer_dock(td, mm_td, sampling_transfer_dock)

    def barrier(self) -> None:
        if self.world_size > 1:
            dist.barrier()

    def wait_all_ref_objs_run_over(self) -> None:
        """Join the non-blocking stages issued so far (all roles, all ranks)."""
        if self._pending and self.overlapping:
            dist.barrier()
        self._pending = 0

    def __getattr__(self, name: str):
        # stage methods: run on the member ranks, skipped elsewhere
        if name.startswith("_") or name in ("worker", "ranks", "is_member"):
            raise AttributeError(name)
        worker = self.__dict__.get("worker")
        if self.__dict__.get("is_member", True):
            if worker is None or not hasattr(worker, name):
                raise AttributeError(name)
            fn = getattr(worker, name)
        else:
            fn = None

        def call(*args, blocking: bool = True, **kwargs):
            out = fn(*args, **kwargs) if fn is not None else None
            if self.overlapping:
                if blocking:
                    dist.barrier()
                else:
                    self._pending += 1
            return out

        return call

    def _from_members(self, value):
        """A value known on the member ranks, made known on all ranks of the job."""
        if self.world_size == 1 or len(self.ranks) == self.world_size:
            return value
        box = [value]
        dist.broadcast_object_list(box, src=self.ranks[0])
        return box[0]

    def save_checkpoint(self, iteration: int) -> None:
        if self.worker is not None:
            self.worker.save_checkpoint(iteration)

    def get_iteration(self) -> int:
        return self._from_members(self.worker.get_iteration() if self.worker is not None else None)

    def get_consumed_train_samples(self) -> int:
        return self._from_members(self.worker.get_consumed_train_samples() if self.worker is not None else None)


def spmd_init(backend: Optional[str] = None, timeout_minutes: int = 30) -> int:
    """Initialise ``torch.distributed`` from the torchrun environment; returns the local rank."""
    import datetime

    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if torch.cuda.is_available():
        torch.cuda.set_device(local_rank)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
        kw = {}
        if backend == "nccl":
            kw["device_id"] = torch.device("cuda", local_rank)
        dist.init_process_group(backend=backend, timeout=datetime.timedelta(minutes=timeout_minutes), **kw)
    return local_rank
