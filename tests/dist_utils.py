"""Multi-process test harness: run a function on ``world_size`` gloo ranks on CPU."""
import os
import socket
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world_size, port, fn, args, errors):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world_size),
                      LOCAL_RANK=str(rank))
    # the ranks share this machine's cores: without a cap every rank starts one thread per core
    torch.set_num_threads(max(1, (os.cpu_count() or world_size) // world_size))
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world_size)
        fn(rank, world_size, *args)
        dist.barrier()
    except Exception:
        errors.put((rank, traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def run_distributed(fn, world_size: int, *args, timeout: float = 300.0):
    """Spawn ``world_size`` processes running ``fn(rank, world_size, *args)``; raises on any failure."""
    ctx = mp.get_context("spawn")
    errors = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_entry, args=(r, world_size, port, fn, args, errors)) for r in range(world_size)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    hung = [p for p in procs if p.is_alive()]
    for p in hung:
        p.terminate()
    if not errors.empty():
        rank, tb = errors.get()
        raise AssertionError(f"rank {rank} failed:\n{tb}")
    assert not hung, "distributed test timed out"
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
