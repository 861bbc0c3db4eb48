"""Parallel state: rank arithmetic and process groups for TP / CP / DP / PP / EP.

Rank order is ``tp-cp-ep-dp-pp`` (TP fastest, PP slowest), the order the reference
initialises Megatron with (``cli/train_grpo.py:657-676``); ``use_tp_pp_dp_mapping`` switches
to ``tp-cp-ep-pp-dp``.  Expert layers re-factor the ``tp*cp*dp`` ranks of a pipeline stage as
``expert_tp * ep * expert_dp``; with ``moe_tp_extend_ep`` the experts are spread over
``tp*ep`` ranks and ``expert_tp = 1``.

All rank lists can be computed without initialising ``torch.distributed`` (``RankLayout``),
which is what the resharding planner and the CPU tests use; ``initialize_model_parallel``
creates the actual process groups (NCCL on GPUs, gloo on CPU).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class RankLayout:
    world_size: int
    tp: int = 1
    pp: int = 1
    cp: int = 1
    ep: int = 1
    moe_tp_extend_ep: bool = False
    tp_pp_dp_order: bool = False

    def __post_init__(self):
        mp = self.tp * self.pp * self.cp
        if self.world_size % mp != 0:
            raise ValueError(f"world size {self.world_size} not divisible by tp*pp*cp = {mp}")
        if self.ep > 1:
            stage = self.world_size // self.pp
            if stage % (self.expert_tp * self.ep_total) != 0:
                raise ValueError("expert parallel size does not divide the ranks of a pipeline stage")

    # sizes ------------------------------------------------------------------------------------
    @property
    def dp(self) -> int:
        return self.world_size // (self.tp * self.pp * self.cp)

    @property
    def expert_tp(self) -> int:
        return 1 if (self.moe_tp_extend_ep or self.ep == 1) else self.tp

    @property
    def ep_total(self) -> int:
        return self.ep * self.tp if self.moe_tp_extend_ep else self.ep

    @property
    def expert_dp(self) -> int:
        return (self.world_size // self.pp) // (self.expert_tp * self.ep_total)

    # coordinates ------------------------------------------------------------------------------
    def _dims(self):
        if self.tp_pp_dp_order:
            return [("tp", self.tp), ("cp", self.cp), ("pp", self.pp), ("dp", self.dp)]
        return [("tp", self.tp), ("cp", self.cp), ("dp", self.dp), ("pp", self.pp)]

    def coords(self, rank: int) -> Dict[str, int]:
        out = {}
        for name, size in self._dims():
            out[name] = rank % size
            rank //= size
        return out

    def rank_of(self, **coord) -> int:
        rank, mult = 0, 1
        for name, size in self._dims():
            rank += coord.get(name, 0) * mult
            mult *= size
        return rank

    def groups(self, *vary: str) -> List[List[int]]:
        """All groups whose members differ only in the dims listed in ``vary``."""
        dims = self._dims()
        fixed = [(n, s) for n, s in dims if n not in vary]
        var = [(n, s) for n, s in dims if n in vary]
        out = []

        def rec(items, cur):
            if not items:
                yield dict(cur)
                return
            (n, s), rest = items[0], items[1:]
            for i in range(s):
                cur[n] = i
                yield from rec(rest, cur)

        for f in rec(fixed, {}):
            members = [self.rank_of(**{**f, **v}) for v in rec(var, {})]
            out.append(sorted(members))
        return out

    # expert view of one pipeline stage --------------------------------------------------------------
    def expert_coords(self, rank: int) -> Dict[str, int]:
        c = self.coords(rank)
        stage_rank = c["tp"] + self.tp * (c["cp"] + self.cp * c["dp"])
        etp, ept = self.expert_tp, self.ep_total
        return {"etp": stage_rank % etp, "ep": (stage_rank // etp) % ept,
                "edp": stage_rank // (etp * ept), "pp": c["pp"]}

    def expert_groups(self, kind: str) -> List[List[int]]:
        """``kind`` in {"ep", "edp", "etp"}."""
        buckets: Dict[tuple, List[int]] = {}
        for r in range(self.world_size):
            c = self.expert_coords(r)
            key = tuple(v for k, v in sorted(c.items()) if k != kind)
            buckets.setdefault(key, []).append(r)
        return [sorted(v) for v in buckets.values()]


class ParallelState:
    """Process groups of one model (actor, critic, ...) living on a set of ranks."""

    def __init__(self, layout: RankLayout, rank: int, backend: Optional[str] = None,
                 rank_offset: int = 0, create_groups: bool = True, timeout=None):
        self.layout = layout
        self.rank = rank                      # rank within the layout (global rank - rank_offset)
        self.rank_offset = rank_offset
        self.backend = backend
        self._groups: Dict[str, Optional[dist.ProcessGroup]] = {}
        self._ranks: Dict[str, List[int]] = {}
        specs = {
            "tp": layout.groups("tp"), "cp": layout.groups("cp"), "pp": layout.groups("pp"),
            "dp": layout.groups("dp"), "dp_cp": layout.groups("dp", "cp"),
            "tp_cp": layout.groups("tp", "cp"), "mp": layout.groups("tp", "pp"),
            "mp_cp": layout.groups("tp", "pp", "cp"),
            "ep": layout.expert_groups("ep"), "edp": layout.expert_groups("edp"),
            "etp": layout.expert_groups("etp"),
        }
        if layout.pp > 1:
            # second group over the pipeline ranks: gradients of the interleaved schedule travel here, so
            # that with two stages (next == previous rank) they cannot be taken for activations
            specs["pp_grad"] = layout.groups("pp")
        # "all": every rank of this model.  When that is the whole job the default group serves.
        inited = dist.is_available() and dist.is_initialized()
        covers_job = inited and rank_offset == 0 and layout.world_size == dist.get_world_size()
        specs["all"] = [list(range(layout.world_size))]
        for name, glist in specs.items():
            for members in glist:
                g = None
                if name == "all" and (covers_job or not inited):
                    pass
                elif create_groups and dist.is_available() and dist.is_initialized() and len(members) > 1:
                    kw = {"timeout": timeout} if timeout is not None else {}
                    g = dist.new_group([m + rank_offset for m in members], backend=backend, **kw)
                if rank in members:
                    self._groups[name] = g
                    self._ranks[name] = members
        self.virtual_pp_rank: Optional[int] = None
        self.virtual_pp_size: Optional[int] = None

    # generic accessors ---------------------------------------------------------------------------
    def group(self, name: str):
        return self._groups.get(name)

    def ranks(self, name: str) -> List[int]:
        return self._ranks[name]

    def global_ranks(self, name: str) -> List[int]:
        return [r + self.rank_offset for r in self._ranks[name]]

    def size(self, name: str) -> int:
        return len(self._ranks[name])

    def rank_in(self, name: str) -> int:
        return self._ranks[name].index(self.rank)

    # Megatron-style getters ---------------------------------------------------------------------
    def get_tensor_model_parallel_group(self): return self.group("tp")
    def get_tensor_model_parallel_world_size(self): return self.size("tp")
    def get_tensor_model_parallel_rank(self): return self.rank_in("tp")
    def get_tensor_model_parallel_src_rank(self): return self.global_ranks("tp")[0]
    def get_pipeline_model_parallel_group(self): return self.group("pp")
    def get_pipeline_model_parallel_world_size(self): return self.size("pp")
    def get_pipeline_model_parallel_rank(self): return self.rank_in("pp")
    def get_pipeline_model_parallel_src_rank(self): return self.global_ranks("pp")[0]
    def get_pipeline_model_parallel_first_rank(self): return self.global_ranks("pp")[0]
    def get_pipeline_model_parallel_last_rank(self): return self.global_ranks("pp")[-1]
    def get_pipeline_model_parallel_next_rank(self):
        r = self.global_ranks("pp"); return r[(self.rank_in("pp") + 1) % len(r)]
    def get_pipeline_model_parallel_prev_rank(self):
        r = self.global_ranks("pp"); return r[(self.rank_in("pp") - 1) % len(r)]
    def is_pipeline_first_stage(self, ignore_virtual: bool = True): return self.rank_in("pp") == 0
    def is_pipeline_last_stage(self, ignore_virtual: bool = True):
        return self.rank_in("pp") == self.size("pp") - 1
    def get_context_parallel_group(self): return self.group("cp")
    def get_context_parallel_world_size(self): return self.size("cp")
    def get_context_parallel_rank(self): return self.rank_in("cp")
    def get_context_parallel_src_rank(self): return self.global_ranks("cp")[0]
    def get_data_parallel_group(self, with_context_parallel: bool = False):
        return self.group("dp_cp" if with_context_parallel else "dp")
    def get_data_parallel_world_size(self, with_context_parallel: bool = False):
        return self.size("dp_cp" if with_context_parallel else "dp")
    def get_data_parallel_rank(self, with_context_parallel: bool = False):
        return self.rank_in("dp_cp" if with_context_parallel else "dp")
    def get_model_parallel_group(self): return self.group("mp")
    def get_expert_model_parallel_group(self): return self.group("ep")
    def get_expert_model_parallel_world_size(self): return self.size("ep")
    def get_expert_model_parallel_rank(self): return self.rank_in("ep")
    def get_expert_data_parallel_group(self): return self.group("edp")
    def get_expert_tensor_parallel_world_size(self): return self.size("etp")
    def get_virtual_pipeline_model_parallel_rank(self): return self.virtual_pp_rank
    def set_virtual_pipeline_model_parallel_rank(self, r): self.virtual_pp_rank = r
    def get_virtual_pipeline_model_parallel_world_size(self): return self.virtual_pp_size


_STATE: Optional[ParallelState] = None


def initialize_model_parallel(tensor_model_parallel_size: int = 1,
                              pipeline_model_parallel_size: int = 1,
                              context_parallel_size: int = 1, expert_model_parallel_size: int = 1,
                              moe_tp_extend_ep: bool = False, use_tp_pp_dp_mapping: bool = False,
                              virtual_pipeline_model_parallel_size: Optional[int] = None,
                              world_size: Optional[int] = None, rank: Optional[int] = None,
                              backend: Optional[str] = None, timeout=None) -> ParallelState:
    """Create the global parallel state (process groups when ``torch.distributed`` is up)."""
    global _STATE
    inited = dist.is_available() and dist.is_initialized()
    ws = world_size if world_size is not None else (dist.get_world_size() if inited else 1)
    rk = rank if rank is not None else (dist.get_rank() if inited else 0)
    layout = RankLayout(ws, tensor_model_parallel_size, pipeline_model_parallel_size,
                        context_parallel_size, expert_model_parallel_size, moe_tp_extend_ep,
                        use_tp_pp_dp_mapping)
    _STATE = ParallelState(layout, rk, backend=backend, timeout=timeout)
    _STATE.virtual_pp_size = virtual_pipeline_model_parallel_size
    return _STATE


def get_parallel_state() -> ParallelState:
    global _STATE
    if _STATE is None:
        _STATE = ParallelState(RankLayout(1), 0, create_groups=False)
    return _STATE


def set_parallel_state(state: Optional[ParallelState]) -> None:
    global _STATE
    _STATE = state


def destroy_model_parallel() -> None:
    set_parallel_state(None)


def model_parallel_is_initialized() -> bool:
    return _STATE is not None
