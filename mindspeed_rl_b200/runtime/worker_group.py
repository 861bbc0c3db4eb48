"""Worker groups: the handle a trainer uses to drive all ranks of one role.

The trainer-facing API is the one of the reference's ``RayActorGroup``
(``mindspeed_rl/workers/scheduler/launcher.py:125-352``): ``initialize``, stage methods with a
``blocking`` flag, ``wait_all_ref_objs_run_over``, ``sync_init_transfer_dock``,
``save_checkpoint``, ``get_iteration``.

``SPMDWorkerGroup`` is the native B200 deployment: one process per GPU launched by
``torchrun``; every process runs the same trainer loop, so a stage call is a plain local call
that all ranks enter together (the collectives inside keep them in lock-step).  Rank 0 is the
*driver*: it owns the experience store (served to the other ranks over ``runtime.rpc``), runs
the CPU stages (rule reward, advantages, metrics, logging) and the others wait at a host
barrier.  ``runtime.launcher`` adds process launching + placement for the single-controller
deployment, and ``RayWorkerGroup`` maps the same calls onto Ray actors when Ray is installed.
"""
from __future__ import annotations

import os
from typing import Any, Callable, List, Optional

import torch
import torch.distributed as dist


class SPMDWorkerGroup:
    def __init__(self, worker, num_gpus: Optional[int] = None):
        self.worker = worker
        inited = dist.is_available() and dist.is_initialized()
        self.rank = dist.get_rank() if inited else 0
        self.world_size = dist.get_world_size() if inited else 1
        self.num_npus = num_gpus or self.world_size
        self.rl_config = getattr(worker, "rl_config", None)
        self.megatron_config = getattr(worker, "actor_config", getattr(worker, "megatron_config", None))
        self.initialized = False
        self._pending: List[Any] = []

    @property
    def is_driver(self) -> bool:
        return self.rank == 0

    def initialize(self):
        self.worker.initialize()
        self.initialized = True
        return self

    def sync_init_transfer_dock(self, td, mm_td=None, sampling_transfer_dock=None) -> None:
        self.worker.init_transfer_dock(td, mm_td, sampling_transfer_dock)

    def barrier(self) -> None:
        if self.world_size > 1:
            dist.barrier()

    def wait_all_ref_objs_run_over(self) -> None:
        self._pending.clear()

    def __getattr__(self, name: str):
        # stage methods: forwarded to the local worker; `blocking` is accepted for API parity
        worker = self.__dict__.get("worker")
        if worker is None or name.startswith("_") or not hasattr(worker, name):
            raise AttributeError(name)
        fn = getattr(worker, name)

        def call(*args, blocking: bool = True, **kwargs):
            return fn(*args, **kwargs)

        return call

    def save_checkpoint(self, iteration: int) -> None:
        self.worker.save_checkpoint(iteration)

    def get_iteration(self) -> int:
        return self.worker.get_iteration()

    def get_consumed_train_samples(self) -> int:
        return self.worker.get_consumed_train_samples()


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
