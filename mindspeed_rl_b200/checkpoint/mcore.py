"""Checkpoints in the Megatron-mcore ``torch`` layout.

    <root>/latest_checkpointed_iteration.txt
    <root>/iter_{iteration:07d}/mp_rank_{tp:02d}[_{pp:03d}][_{ep:03d}]/model_optim_rng.pt
    <root>/iter_{iteration:07d}/mp_rank_.../distrib_optim.pt          (distributed optimizer shard)

``model_optim_rng.pt`` holds ``{'args', 'checkpoint_version', 'iteration', 'model' (or 'model0'..
for virtual pipeline chunks), 'optimizer', 'opt_param_scheduler', 'rng_state',
'num_floating_point_operations_so_far'}``; parameter names are the mcore names used throughout
the framework (``decoder.layers.N.self_attention.linear_qkv.weight`` ...).  Layer indices inside a
pipeline stage are local (0-based per stage), as in Megatron.  With data-parallel size > 1 the
optimizer shard of DP rank ``r > 0`` goes to ``distrib_optim_{r:03d}.pt`` next to rank 0's file.

Load honours ``finetune`` (weights only, iteration reset), ``no_load_optim``, ``no_load_rng`` and
``load_checkpoint_loosely`` (non-strict key matching).  Reference call sites:
``workers/actor_hybrid_worker.py:365-379``, ``workers/integrated_worker.py:226-261``.
"""
from __future__ import annotations

import os
import random
import re
from types import SimpleNamespace
from typing import Any, Dict, List, Optional, Tuple

import numpy as np
import torch

TRACKER = "latest_checkpointed_iteration.txt"
CHECKPOINT_VERSION = 3.0


def checkpoint_dir(root: str, iteration: int, release: bool = False) -> str:
    return os.path.join(root, "release" if release else f"iter_{iteration:07d}")


def rank_dir_name(tp_rank: int, pp_rank: int = 0, pp_size: int = 1, ep_rank: int = 0, ep_size: int = 1) -> str:
    name = f"mp_rank_{tp_rank:02d}"
    if pp_size > 1:
        name += f"_{pp_rank:03d}"
    if ep_size > 1:
        name += f"_{ep_rank:03d}"
    return name


def _coords(ps) -> Tuple[int, int, int, int, int, int]:
    # With expert parallelism the EP ranks are carved out of the data-parallel group and each holds
    # different experts: every EP rank has a directory of its own, and inside it the replicas are
    # told apart by the expert-data-parallel rank (replica 0 writes the model file, as Megatron does
    # with ``expert_data_parallel_rank == 0``).  Dense-only models use the data-parallel rank.
    ep_size = ps.size("ep")
    replica = ps.rank_in("edp") if ep_size > 1 else ps.rank_in("dp_cp")
    return (ps.rank_in("tp"), ps.rank_in("pp"), ps.size("pp"), ps.rank_in("ep"), ep_size, replica)


def read_tracker(root: str) -> Tuple[Optional[int], bool]:
    path = os.path.join(root, TRACKER)
    if not os.path.isfile(path):
        return None, False
    text = open(path).read().strip()
    if text == "release":
        return 0, True
    return int(text), False


def _to_local_names(state: Dict[str, torch.Tensor], layer_numbers: List[int]) -> Dict[str, torch.Tensor]:
    """Global layer numbers -> per-stage local indices (module list order)."""
    return state  # the module list is already indexed locally (0..n_local-1)


def _rng_state() -> Dict[str, Any]:
    st = {"random_rng_state": random.getstate(), "np_rng_state": np.random.get_state(),
          "torch_rng_state": torch.get_rng_state()}
    if torch.cuda.is_available():
        st["cuda_rng_state"] = torch.cuda.get_rng_state()
    return st


def _restore_rng(st: Dict[str, Any]) -> None:
    random.setstate(st["random_rng_state"])
    np.random.set_state(st["np_rng_state"])
    torch.set_rng_state(st["torch_rng_state"])
    if torch.cuda.is_available() and "cuda_rng_state" in st:
        torch.cuda.set_rng_state(st["cuda_rng_state"])


def save_checkpoint(root: str, iteration: int, model, optimizer=None, opt_param_scheduler=None, ps=None,
                    config=None, num_floating_point_operations_so_far: float = 0.0,
                    consumed_train_samples: int = 0, models: Optional[List[Any]] = None) -> str:
    """Write this rank's part of the checkpoint; returns the rank directory."""
    from ..parallel.state import get_parallel_state

    ps = ps or get_parallel_state()
    tp, pp, pp_size, ep, ep_size, dp = _coords(ps)
    d = os.path.join(checkpoint_dir(root, iteration), rank_dir_name(tp, pp, pp_size, ep, ep_size))
    os.makedirs(d, exist_ok=True)
    if dp == 0:
        args = SimpleNamespace(**(dict(config.dict()) if config is not None and hasattr(config, "dict") else {}))
        args.iteration = iteration
        args.consumed_train_samples = consumed_train_samples
        state: Dict[str, Any] = {"args": args, "checkpoint_version": CHECKPOINT_VERSION, "iteration": iteration,
                                 "num_floating_point_operations_so_far": num_floating_point_operations_so_far,
                                 "rng_state": [_rng_state()]}
        chunks = models if models is not None else [model]
        if len(chunks) == 1:
            state["model"] = {k: v.detach().cpu() for k, v in chunks[0].state_dict().items()}
        else:
            for i, m in enumerate(chunks):
                state[f"model{i}"] = {k: v.detach().cpu() for k, v in m.state_dict().items()}
        if optimizer is not None and not getattr(config, "no_save_optim", False):
            state["optimizer"] = {"step": optimizer.step_count, "param_groups": optimizer.param_groups}
        if opt_param_scheduler is not None:
            state["opt_param_scheduler"] = opt_param_scheduler.state_dict()
        torch.save(state, os.path.join(d, "model_optim_rng.pt"))
    if optimizer is not None and not getattr(config, "no_save_optim", False):
        name = "distrib_optim.pt" if dp == 0 else f"distrib_optim_{dp:03d}.pt"
        torch.save(optimizer.state_dict(), os.path.join(d, name))
    _barrier()
    if _is_rank0():
        with open(os.path.join(root, TRACKER), "w") as fh:
            fh.write(str(iteration))
    _barrier()
    return d


def load_checkpoint(root: str, model, optimizer=None, opt_param_scheduler=None, ps=None, config=None,
                    strict: bool = True, iteration: Optional[int] = None,
                    models: Optional[List[Any]] = None) -> Tuple[int, int]:
    """Load this rank's part. Returns ``(iteration, consumed_train_samples)`` (zeros when
    fine-tuning or when no checkpoint exists)."""
    from ..parallel.state import get_parallel_state

    ps = ps or get_parallel_state()
    release = False
    if iteration is None:
        iteration, release = read_tracker(root)
        if iteration is None:
            return 0, 0
    tp, pp, pp_size, ep, ep_size, dp = _coords(ps)
    d = os.path.join(checkpoint_dir(root, iteration, release), rank_dir_name(tp, pp, pp_size, ep, ep_size))
    path = os.path.join(d, "model_optim_rng.pt")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"checkpoint file not found: {path}")
    state = torch.load(path, map_location="cpu", weights_only=False)
    loosely = bool(getattr(config, "load_checkpoint_loosely", False)) or not strict
    chunks = models if models is not None else [model]
    for i, m in enumerate(chunks):
        sd = state["model"] if len(chunks) == 1 else state[f"model{i}"]
        if getattr(config, "lora_ckpt_filter", False):
            sd = {k: v for k, v in sd.items() if "lora_" in k}
            loosely = True
        missing, unexpected = m.load_state_dict(sd, strict=False)
        if not loosely and (missing or unexpected):
            raise RuntimeError(f"checkpoint mismatch: missing {missing[:5]}, unexpected {unexpected[:5]}")
    finetune = bool(getattr(config, "finetune", False))
    if finetune:
        if optimizer is not None:
            optimizer.reload_model_params()
        return 0, 0
    if optimizer is not None and not getattr(config, "no_load_optim", False):
        name = "distrib_optim.pt" if dp == 0 else f"distrib_optim_{dp:03d}.pt"
        opath = os.path.join(d, name)
        if os.path.isfile(opath):
            optimizer.load_state_dict(torch.load(opath, map_location="cpu", weights_only=False))
        else:
            optimizer.reload_model_params()
        if opt_param_scheduler is not None and "opt_param_scheduler" in state:
            opt_param_scheduler.load_state_dict(state["opt_param_scheduler"])
    elif optimizer is not None:
        optimizer.reload_model_params()
    if not getattr(config, "no_load_rng", False) and state.get("rng_state"):
        try:
            _restore_rng(state["rng_state"][0])
        except Exception:
            pass
    args = state.get("args")
    return int(state.get("iteration", 0)), int(getattr(args, "consumed_train_samples", 0) or 0)


def load_args_from_checkpoint(root: str) -> Optional[SimpleNamespace]:
    it, release = read_tracker(root)
    if it is None:
        return None
    base = checkpoint_dir(root, it, release)
    for name in sorted(os.listdir(base)):
        p = os.path.join(base, name, "model_optim_rng.pt")
        if os.path.isfile(p):
            return torch.load(p, map_location="cpu", weights_only=False).get("args")
    return None


def _is_rank0() -> bool:
    import torch.distributed as dist

    return not (dist.is_available() and dist.is_initialized()) or dist.get_rank() == 0


def _barrier() -> None:
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()
