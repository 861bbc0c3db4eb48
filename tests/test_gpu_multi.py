"""Multi-GPU tests (skipped on boxes with a single GPU): peer-memory collectives, the reshard
copy-plan kernel and a GRPO iteration with train TP != rollout TP, each run as one process per
GPU under ``torch.distributed.run``."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _n_gpus() -> int:
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _free_port() -> int:
    import socket

    with socket.socket() as s:          # two test runs on one box must not meet on a fixed port
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(case: str, nproc: int, timeout: int = 600) -> str:
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(ROOT, "tests", "multi_gpu_cases.py"), case]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    out = res.stdout + res.stderr
    assert res.returncode == 0 and f"CASE {case} OK" in out, out[-4000:]
    return out


@pytest.mark.skipif(_n_gpus() < 2, reason="needs at least 2 GPUs")
def test_symmetric_collectives():
    _run("collectives", min(_n_gpus(), 8))


@pytest.mark.skipif(_n_gpus() < 2, reason="needs at least 2 GPUs")
def test_reshard_copy_plan_kernel():
    _run("reshard", 2)
    if _n_gpus() >= 4:
        _run("reshard", 4)


@pytest.mark.skipif(_n_gpus() < 2, reason="needs at least 2 GPUs")
def test_grpo_train_tp2_rollout_tp1():
    _run("grpo_reshard", 2)


@pytest.mark.skipif(_n_gpus() < 2, reason="needs at least 2 GPUs")
def test_fused_tp_kernels():
    _run("fused_tp", 2)
    if _n_gpus() >= 4:
        _run("fused_tp", 4)


@pytest.mark.skipif(_n_gpus() < 2, reason="needs at least 2 GPUs")
def test_moe_expert_parallel():
    _run("moe_ep", 2)
    _run("moe_ep_p2p", 2)


@pytest.mark.skipif(_n_gpus() < 2, reason="needs at least 2 GPUs")
def test_ring_attention_context_parallel():
    _run("cp_ring", 2)


@pytest.mark.skipif(_n_gpus() < 2, reason="needs at least 2 GPUs")
def test_arena_setup_failure_is_collective():
    _run("arena_fallback", 2)


@pytest.mark.skipif(_n_gpus() < 2, reason="needs at least 2 GPUs")
def test_tp_model_with_fused_linears():
    _run("tp_model", 2)


@pytest.mark.skipif(_n_gpus() < 2, reason="needs at least 2 GPUs")
def test_peer_memory_all_reduce_for_decode():
    _run("peer_all_reduce", 2)
    if _n_gpus() >= 4:
        _run("peer_all_reduce", 4)


@pytest.mark.skipif(_n_gpus() < 2, reason="needs at least 2 GPUs")
def test_releasable_peer_mapped_buffers():
    _run("buffer_release", 2)


@pytest.mark.skipif(_n_gpus() < 2, reason="needs at least 2 GPUs")
def test_overlapped_grad_reduce_and_pipelined_param_gather():
    _run("overlap", 2)
