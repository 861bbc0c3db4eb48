"""Per-GPU worker base: data-plane access shared by every role.

Each model-parallel replica has one *leader* (tp 0, cp 0, pp 0) that talks to the experience
store; what it pulls is fanned out to the other ranks of the replica in **one** host-side
object broadcast (header + payload together), and results are written back only by the last
pipeline stage's tp-0 rank.  This replaces the per-column broadcast cascades of the reference
(``mindspeed_rl/workers/base_worker.py:367-516,685-822``) while keeping its semantics: ragged
rows from the store arrive as padded 2-D tensors, padded to a multiple of ``tp*cp`` (``2*tp*cp``
for ring context parallel).
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..obs.profiler import nvtx_range, profiler_start, profiler_stop
from ..parallel.state import ParallelState, get_parallel_state
from ..utils.device_status import check_device_status
from ..utils.pad_process import (pad_rows, padding_dict_to_tensor_dict,
                                 remove_padding_tensor_dict_to_dict, truncate_rows)

_TOKEN_COLUMNS = ("prompts", "responses", "input_ids", "labels")


def pad_batch(ragged: Dict[str, List[torch.Tensor]], pad_id: int, multiple: int = 1) -> Dict[str, torch.Tensor]:
    """Ragged rows -> ``[n, W]`` tensors; 1-element columns become ``[n]``."""
    out = {}
    for k, rows in ragged.items():
        rows = list(rows)
        if k in _TOKEN_COLUMNS:
            out[k] = pad_rows(rows, pad_id, multiple).long()
        elif all(r.numel() == 1 for r in rows):
            out[k] = torch.stack([r.reshape(()) for r in rows])
        else:
            out[k] = pad_rows(rows, 0)
    return out


def _align_mm(mm, cols):
    """One dict per sample with the per-prompt items of the requested columns (``None`` for fillers)."""
    names = list(cols)
    out, k = [], 0
    for m in mm:
        if m is None:
            out.append(None)
            continue
        out.append({c: cols[c][k] for c in names})
        k += 1
    return out


def profiled_stage(role: str):
    """Wrap a worker stage with an NVTX range and, when the run's profiler config selects this
    rank / stage / iteration, a ``torch.profiler`` session (reference hook sites:
    ``workers/actor_hybrid_worker.py:309-313,428-429,819-823``)."""
    def deco(fn):
        import functools

        @functools.wraps(fn)
        def wrapped(self, *a, **kw):
            prof = profiler_start(getattr(self, "profiler_config", None), role,
                                  getattr(self, "iteration", None))
            dump = getattr(self, "tensor_dump", None)
            try:
                with nvtx_range(role):
                    out = fn(self, *a, **kw)
                check_device_status(role)
                return out
            finally:
                profiler_stop(prof)
                if dump is not None and role in ("actor_update", "critic_update"):
                    dump.step()
        return wrapped
    return deco


class BaseWorker:
    def __init__(self, td=None, pad_token_id: int = 0, state: Optional[ParallelState] = None):
        self.td = td
        self.pad_token_id = pad_token_id
        self._state = state

    # ---- parallel coordinates ------------------------------------------------------------------
    @property
    def parallel_state(self) -> ParallelState:
        return self._state or get_parallel_state()

    def is_replica_leader(self, tp_rank=None, cp_rank=None, pp_rank=None) -> bool:
        ps = self.parallel_state
        return ps.rank_in("tp") == 0 and ps.rank_in("cp") == 0 and ps.rank_in("pp") == 0

    def is_writer(self) -> bool:
        ps = self.parallel_state
        return ps.rank_in("tp") == 0 and ps.rank_in("cp") == 0 and ps.is_pipeline_last_stage()

    def _replica_group(self):
        ps = self.parallel_state
        return ps.group("mp_cp"), ps.global_ranks("mp_cp")[0], ps.size("mp_cp")

    def _side_channel(self, group, src: int, size: int):
        """ZeroMQ broadcast channel of this replica (``rl_config.zmq_communication``), created on
        first use by all members together; ``None`` when the option is off."""
        rl = getattr(self, "rl_config", None)
        if rl is None or not getattr(rl, "zmq_communication", False):
            return None
        cache = self.__dict__.setdefault("_side_channels", {})
        key = id(group)
        if key not in cache:
            from ..runtime.zmq_broadcast import setup_replica_broadcast

            cache[key] = setup_replica_broadcast(group, src, size, self.is_replica_leader())
        return cache[key]

    # ---- data plane ------------------------------------------------------------------------------
    def dispatch_transfer_dock_data(self, consumer: str, columns: Sequence[str], experience_count: int,
                                    pad_multiple: int = 1, indexes: Optional[List[int]] = None,
                                    get_n_samples: bool = True, use_batch_seqlen_balance: bool = False,
                                    dp_size: int = 1, mm_columns: Optional[Sequence[str]] = None
                                    ) -> Tuple[Optional[Dict[str, torch.Tensor]], Optional[List[int]], bool]:
        """Returns ``(batch, indexes, finished)``.  ``finished`` is True when the consumer has
        nothing left to process in this iteration (then ``batch`` is ``None``).  ``mm_columns``: per-prompt
        columns of the multimodal store to attach as ``batch["mm"]`` (one dict per sample)."""
        group, src, size = self._replica_group()
        payload = None
        if self.is_replica_leader():
            if self.td.all_consumed(consumer):
                payload = (None, None, True)
            else:
                batch, idx = self.td.get_experience(consumer, list(columns), experience_count,
                                                    dp_size=dp_size, indexes=indexes,
                                                    get_n_samples=get_n_samples,
                                                    use_batch_seqlen_balance=use_batch_seqlen_balance)
                mm = None
                mm_td = getattr(self, "mm_td", None)
                if mm_columns and mm_td is not None and idx:
                    cols = mm_td.get_experience_dict(list(mm_columns), [i for i in idx if i >= 0], get_n_samples=False)
                    mm = _align_mm([({} if i >= 0 else None) for i in idx], cols)
                payload = (batch, idx, False, mm)
        if payload is not None and len(payload) == 3:
            payload = payload + (None,)
        if size > 1 and dist.is_initialized():
            channel = self._side_channel(group, src, size)
            if channel is not None:          # host-side ZeroMQ fan-out, no collective on the device stream
                payload = channel.broadcast(payload)
            else:
                box = [payload]
                dist.broadcast_object_list(box, src=src, group=group)
                payload = box[0]
        batch, idx, finished, mm = payload
        if finished or not batch or not idx:
            return None, None, finished
        ragged = remove_padding_tensor_dict_to_dict(batch)
        out = pad_batch(ragged, self.pad_token_id, pad_multiple)
        if mm is not None:
            out["mm"] = mm
        return out, idx, False

    def collect_transfer_dock_data(self, output: Dict[str, torch.Tensor], indexes: List[int],
                                   lengths: Optional[torch.Tensor] = None) -> None:
        """Write result columns back (ragged when ``lengths`` is given). Only one rank per replica
        writes."""
        if not self.is_writer():
            return
        out = {}
        for k, v in output.items():
            if isinstance(v, list):
                out[k] = [t.detach().cpu() for t in v]
            elif lengths is not None and v.dim() == 2 and v.shape[1] > 1:
                out[k] = truncate_rows(v.detach().cpu(), lengths)
            else:
                out[k] = [row.reshape(-1) for row in v.detach().cpu()]
        self.td.put_experience(padding_dict_to_tensor_dict(out), indexes)

    def dump_key_data(self, stage: str, switch: str, tensors: Dict[str, Any]) -> None:
        """Statistics of a stage's key tensors for the accuracy-debugging dump (``msprobe_config``: prompts,
        responses, log-probs, advantages, losses; reference call sites ``actor_hybrid_worker.py:315,349-350,573``,
        ``grpo_actor_loss_func.py:81-89``).  Only the writer rank of a replica records."""
        dump = getattr(self, "tensor_dump", None)
        if dump is None or not dump.wants(switch) or not self.is_writer():
            return
        flat = {}
        for k, v in tensors.items():
            if isinstance(v, (list, tuple)) and v and torch.is_tensor(v[0]):
                v = torch.cat([t.reshape(-1).float() for t in v])
            flat[k] = v
        dump.save_data(stage, flat)

    def update_metrics(self, key, value, cumulate=True) -> None:
        if self.is_writer():
            self.td.update_metrics(key, value=value, cumulate=cumulate)
