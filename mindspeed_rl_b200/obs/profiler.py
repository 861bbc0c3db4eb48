"""Stage profiling, range markers, tensor dumps, seeding and FLOP accounting.

* ``profiler_start / profiler_step / profiler_stop``: a ``torch.profiler`` session (CPU + CUDA
  activities) for one worker stage, selected by rank, stage name and iteration window from
  ``ProfilerConfig`` exactly as the reference selects its device profiler
  (``mindspeed_rl/utils/utils.py:518-638``; keys ``profile, stage, profile_ranks,
  profile_step_start/end, profile_level, profile_with_memory/cpu/module, profile_record_shapes,
  profile_save_path, profile_export_type``).  Traces land under ``<save_path>/<role>``.
* ``range_timer`` / ``nvtx_range``: the light-weight markers wrapped around stage functions,
  reshard and offload steps (reference decorator ``mstx_timer_decorator``, ``utils.py:594-601``);
  NVTX ranges on CUDA builds, no-ops elsewhere; active only when ``mstx`` is configured.
* ``TensorDump``: step/stage-scoped dump of named tensors' statistics (and optionally values) for
  accuracy comparison between runs (role of the reference's msprobe hooks, ``utils.py:384-490``).
* ``seed_all``: python / numpy / torch seeding plus deterministic-algorithm switches
  (``utils.py:321-333``).
* ``num_floating_point_operations``: model FLOPs per batch for throughput reporting
  (``utils.py:195-303``).
"""
from __future__ import annotations

import contextlib
import functools
import json
import os
import random
from typing import Any, Dict, Iterable, List, Optional

import numpy as np
import torch

_MSTX_ON = False


def enable_range_markers(on: bool = True) -> None:
    global _MSTX_ON
    _MSTX_ON = bool(on)


@contextlib.contextmanager
def nvtx_range(name: str):
    live = _MSTX_ON and torch.cuda.is_available()
    if live:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if live:
            torch.cuda.nvtx.range_pop()


def range_timer(fn):
    """Decorator: NVTX range named after the function (when range markers are enabled)."""
    @functools.wraps(fn)
    def wrapped(*a, **kw):
        with nvtx_range(fn.__qualname__):
            return fn(*a, **kw)
    return wrapped


# ---- torch.profiler sessions -----------------------------------------------------------------------
def _rank() -> int:
    import torch.distributed as dist

    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def _selected(cfg, role: str, iteration: Optional[int]) -> bool:
    if cfg is None or not getattr(cfg, "profile", False):
        return False
    ranks = getattr(cfg, "profile_ranks", "all")
    if ranks != "all" and _rank() not in list(ranks or []):
        return False
    stage = getattr(cfg, "stage", "all")
    if stage != "all":
        stages = [stage] if isinstance(stage, str) else list(stage)
        if role not in stages:
            return False
    if iteration is not None:
        lo, hi = getattr(cfg, "profile_step_start", 1), getattr(cfg, "profile_step_end", 2)
        if not (lo <= iteration < hi):
            return False
    return True


def profiler_start(cfg, role: str = "profiler_data", profiler_iteration: Optional[int] = None):
    """Started ``torch.profiler.profile`` for this stage, or ``None`` when not selected."""
    if not _selected(cfg, role, profiler_iteration):
        return None
    from torch.profiler import ProfilerActivity, profile, schedule, tensorboard_trace_handler

    acts = [ProfilerActivity.CPU] if (getattr(cfg, "profile_with_cpu", True) or not torch.cuda.is_available()) else []
    if torch.cuda.is_available():
        acts.append(ProfilerActivity.CUDA)
    level = str(getattr(cfg, "profile_level", "level0"))
    out_dir = os.path.join(getattr(cfg, "profile_save_path", "./profiler_data") or "./profiler_data", role)
    os.makedirs(out_dir, exist_ok=True)
    if getattr(cfg, "profile_export_type", "text") == "db":
        handler = lambda p: p.export_chrome_trace(os.path.join(out_dir, f"trace_rank{_rank()}_{p.step_num}.json"))
    else:
        handler = tensorboard_trace_handler(out_dir)
    sched = None
    if profiler_iteration is None:
        skip = max(getattr(cfg, "profile_step_start", 1) - 1, 0)
        active = max(getattr(cfg, "profile_step_end", 2) - getattr(cfg, "profile_step_start", 1), 1)
        sched = schedule(wait=0, warmup=0, active=active, repeat=1, skip_first=skip)
    prof = profile(activities=acts, schedule=sched, on_trace_ready=handler,
                   record_shapes=bool(getattr(cfg, "profile_record_shapes", False)),
                   profile_memory=bool(getattr(cfg, "profile_with_memory", False)),
                   with_stack=level in ("level2", "2"),
                   with_modules=bool(getattr(cfg, "profile_with_module", False)))
    prof.start()
    return prof


def profiler_step(prof) -> None:
    if prof is not None:
        prof.step()


def profiler_stop(prof) -> None:
    if prof is not None:
        prof.stop()


# ---- tensor dumps ---------------------------------------------------------------------------------------
class TensorDump:
    """Collect named tensors per (iteration, stage) and write ``<dump_path>/step{N}/rank{R}/<stage>.json``
    (+ ``.pt`` with the values when ``save_values``).  Keys of ``MsprobeConfig`` that map here:
    ``msprobe`` (on/off), ``dump_path``, ``key_data_dump`` (statistics of stage inputs/outputs),
    ``configurations_dump``, ``step_start/step_end``."""

    def __init__(self, cfg=None, *, enabled: Optional[bool] = None, dump_path: Optional[str] = None,
                 save_values: bool = False):
        self.enabled = bool(getattr(cfg, "msprobe", False)) if enabled is None else enabled
        self.dump_path = dump_path or getattr(cfg, "dump_path", "./msprobe_dump") or "./msprobe_dump"
        self.key_data = bool(getattr(cfg, "key_data_dump", True)) if cfg is not None else True
        # per-stage switches (``actor_train_dump`` ...): when none is set, ``key_data_dump`` covers every stage
        names = ("actor_train_dump", "actor_infer_dump", "reference_dump", "critic_train_dump")
        chosen = {n for n in names if bool(getattr(cfg, n, False))} if cfg is not None else set()
        self.stages = chosen or set(names)
        self.lo = getattr(cfg, "step_start", 0) if cfg is not None else 0
        self.hi = getattr(cfg, "step_end", 1 << 30) if cfg is not None else 1 << 30
        self.save_values = save_values
        self.iteration = 0
        self._records: Dict[str, Dict[str, Any]] = {}
        self._values: Dict[str, Dict[str, torch.Tensor]] = {}

    def active(self) -> bool:
        return self.enabled and self.lo <= self.iteration <= self.hi

    @staticmethod
    def stats(t: torch.Tensor) -> Dict[str, Any]:
        f = t.detach().float()
        if f.numel() == 0:
            return {"shape": list(t.shape), "dtype": str(t.dtype), "numel": 0}
        return {"shape": list(t.shape), "dtype": str(t.dtype), "numel": t.numel(), "mean": float(f.mean()),
                "absmax": float(f.abs().max()), "min": float(f.min()), "max": float(f.max()),
                "l2": float(f.norm()), "nan": int(torch.isnan(f).sum()), "inf": int(torch.isinf(f).sum())}

    def wants(self, switch: str) -> bool:
        return self.active() and self.key_data and switch in self.stages

    def save_data(self, stage: str, tensors: Dict[str, Any]) -> None:
        if not (self.active() and self.key_data):
            return
        rec = self._records.setdefault(stage, {})
        for k, v in tensors.items():
            if torch.is_tensor(v):
                rec[k] = self.stats(v)
                if self.save_values:
                    self._values.setdefault(stage, {})[k] = v.detach().cpu()
            elif isinstance(v, (int, float, str, bool)) or v is None:
                rec[k] = v

    def save_configs(self, configs: Dict[str, Any]) -> None:
        if not self.enabled:
            return
        os.makedirs(self.dump_path, exist_ok=True)
        plain = {k: (v.dict() if hasattr(v, "dict") else getattr(v, "__dict__", str(v))) for k, v in configs.items()}
        with open(os.path.join(self.dump_path, "configurations.json"), "w") as fh:
            json.dump(plain, fh, indent=1, default=str)

    def step(self) -> None:
        """Flush this iteration's records and move on."""
        if self.active() and self._records:
            d = os.path.join(self.dump_path, f"step{self.iteration}", f"rank{_rank()}")
            os.makedirs(d, exist_ok=True)
            for stage, rec in self._records.items():
                with open(os.path.join(d, f"{stage}.json"), "w") as fh:
                    json.dump(rec, fh, indent=1)
                if stage in self._values:
                    torch.save(self._values[stage], os.path.join(d, f"{stage}.pt"))
        self._records, self._values = {}, {}
        self.iteration += 1


# ---- determinism -------------------------------------------------------------------------------------------
def seed_all(seed: int = 1234, deterministic: bool = False) -> None:
    random.seed(seed)
    os.environ["PYTHONHASHSEED"] = str(seed)
    np.random.seed(seed % (1 << 32))
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
    if deterministic:
        os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")
        os.environ.setdefault("NCCL_ALGO", "Ring")          # fixed reduction order across runs
        torch.use_deterministic_algorithms(True, warn_only=True)
        torch.backends.cudnn.deterministic = True
        torch.backends.cudnn.benchmark = False


# ---- FLOP accounting ----------------------------------------------------------------------------------------
def num_floating_point_operations(cfg, batch_size: int, seq_length: Optional[int] = None) -> float:
    """Forward + backward FLOPs of a decoder for ``batch_size`` sequences of ``seq_length`` tokens
    (3x the forward matmul FLOPs; causal attention counted at half the dense score cost is NOT
    applied, matching the usual Megatron accounting)."""
    s = seq_length or getattr(cfg, "seq_length", None) or getattr(cfg, "max_position_embeddings")
    h, layers = cfg.hidden_size, cfg.num_layers
    nh = cfg.num_attention_heads
    nkv = getattr(cfg, "num_query_groups", None) or nh
    hd = getattr(cfg, "kv_channels", None) or h // nh
    ffn = cfg.ffn_hidden_size
    vocab = getattr(cfg, "padded_vocab_size", None) or getattr(cfg, "vocab_size")
    n_exp = getattr(cfg, "num_experts", None) or 0
    topk = getattr(cfg, "moe_router_topk", 1) if n_exp else 1
    moe_ffn = getattr(cfg, "moe_ffn_hidden_size", None) or ffn
    shared = (getattr(cfg, "n_shared_experts", None) or 0) * moe_ffn if n_exp else 0
    dense_first = getattr(cfg, "first_k_dense_replace", 0) or 0 if n_exp else layers
    glu = 3 if getattr(cfg, "swiglu", True) else 2
    per_tok_attn = 2 * h * (nh * hd + 2 * nkv * hd) + 2 * nh * hd * h + 2 * 2 * s * nh * hd
    per_tok_dense = 2 * glu * h * ffn
    per_tok_moe = 2 * glu * h * (moe_ffn * topk + shared) + 2 * h * n_exp
    n_moe = max(layers - dense_first, 0) if n_exp else 0
    per_tok = layers * per_tok_attn + (layers - n_moe) * per_tok_dense + n_moe * per_tok_moe + 2 * h * vocab
    return 3.0 * batch_size * s * per_tok
