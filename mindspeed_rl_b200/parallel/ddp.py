"""Contiguous parameter / gradient buffers and data-parallel gradient reduction.

Every trainable parameter of a model chunk becomes a view into one flat ``param_data`` buffer
and gets a ``main_grad`` view into a matching ``grad_data`` buffer (bf16, or fp32 with
``accumulate_allreduce_grads_in_fp32``).  The layer backward accumulates straight into
``main_grad``.  The flat layout is what makes whole-model operations single kernels or single
collectives: gradient reduce-scatter / all-reduce over DP, the Adam update, the parameter
all-gather of the distributed optimizer, offload to pinned host memory and the train->rollout
resharding plan.

Role in the reference: Megatron's ``DistributedDataParallel`` with ``use_distributed_optimizer``
(``mindspeed_rl/workers/resharding/megatron_off_loader.py:138-224`` walks the same buffers).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn


def _align(n: int, a: int) -> int:
    return (n + a - 1) // a * a


@dataclass
class ParamSlot:
    name: str
    start: int
    numel: int
    shape: torch.Size


class ParamAndGradBuffer:
    """Flat storage of the trainable parameters of one model chunk."""

    ALIGN = 64  # elements; keeps every parameter 128-byte aligned in bf16

    def __init__(self, named_params: Iterable[Tuple[str, nn.Parameter]], dp_size: int = 1,
                 grad_dtype: Optional[torch.dtype] = None, bucket_numel: Optional[int] = None,
                 group=None, dp_rank: Optional[int] = None, grad_scale: Optional[float] = None,
                 is_expert: bool = False, releasable_params: bool = False, releasable_grads: bool = False,
                 with_grads: bool = True):
        # ``group`` / ``dp_rank`` / ``dp_size``: the ranks that hold replicas of these parameters.
        # Dense parameters are replicated over the whole data-parallel group; expert parameters
        # only over the expert-data-parallel group (the EP ranks hold different experts), but their
        # gradient average still runs over all data-parallel ranks' tokens (``grad_scale``).
        self.group, self.is_expert = group, is_expert
        self.dp_rank = dp_rank if dp_rank is not None else (
            dist.get_rank(group) if (group is not None and dist.is_initialized()) else 0)
        self.grad_scale = grad_scale if grad_scale is not None else 1.0 / max(dp_size, 1)
        # ``with_grads=False``: a parameter-only buffer for frozen weights (the base weights under LoRA), so
        # that they too sit in peer-mapped memory where the rollout resharding can read them
        self.with_grads = with_grads
        params = [(n, p) for n, p in named_params if p.requires_grad or not with_grads]
        if not params:
            raise ValueError("no trainable parameters")
        self.param_dtype = params[0][1].dtype
        self.device = params[0][1].device
        if any(p.dtype != self.param_dtype for _, p in params):
            raise ValueError("all buffered parameters must share one dtype")
        self.grad_dtype = grad_dtype or self.param_dtype
        self.dp_size = dp_size
        self.slots: List[ParamSlot] = []
        off = 0
        for n, p in params:
            self.slots.append(ParamSlot(n, off, p.numel(), p.shape))
            off = _align(off + p.numel(), self.ALIGN)
        self.numel = _align(off, self.ALIGN * max(dp_size, 1))
        # With a symmetric arena the flat buffers are peer-mapped: gradient reduce-scatter,
        # parameter all-gather and rollout resharding then run as direct NVLink pull kernels.
        # A buffer marked releasable gets a peer-mapped segment of its own (same team as the arena)
        # instead of a slice of the job-wide arena, so that it can be unmapped and freed while the
        # rollout needs the memory and mapped again afterwards (``release_*`` / ``restore_*``).
        self.param_arena = self.grad_arena = None
        self._own = {"param": False, "grad": False}
        self._team = None
        if self.device.type == "cuda":
            from .symm import get_arena

            arena = get_arena()
            if arena is not None:
                self._team = arena.group
                p_bytes = self.numel * torch.empty(0, dtype=self.param_dtype).element_size() + 512
                g_bytes = self.numel * torch.empty(0, dtype=self.grad_dtype).element_size() + 512
                if releasable_params:
                    self.param_arena = self._segment(p_bytes)
                    self._own["param"] = self.param_arena is not None
                if releasable_grads and with_grads:
                    self.grad_arena = self._segment(g_bytes)
                    self._own["grad"] = self.grad_arena is not None
                want_g = with_grads and not releasable_grads
                shared = (0 if releasable_params else p_bytes) + (g_bytes if want_g else 0)
                if shared and arena.free_bytes() >= shared:
                    if not releasable_params:
                        self.param_arena = arena
                    if want_g:
                        self.grad_arena = arena
        self.param_data = self._new_flat(self.param_arena, self.param_dtype)
        self.grad_data = self._new_flat(self.grad_arena, self.grad_dtype) if with_grads else \
            torch.empty(0, dtype=self.grad_dtype, device=self.device)
        self.params: List[nn.Parameter] = []
        for (n, p), slot in zip(params, self.slots):
            view = self.param_data[slot.start:slot.start + slot.numel].view(slot.shape)
            view.copy_(p.data)
            p.data = view
            if with_grads:
                p.main_grad = self.grad_data[slot.start:slot.start + slot.numel].view(slot.shape)
                p.grad = None
            self.params.append(p)
        self.by_name: Dict[str, ParamSlot] = {s.name: s for s in self.slots}

    # ---- storage -------------------------------------------------------------------------------------
    @property
    def arena(self):
        """A peer-mapped home of (one of) the flat buffers, or ``None`` when both are plain allocations."""
        return self.param_arena if self.param_arena is not None else self.grad_arena

    def _segment(self, nbytes: int):
        """A peer-mapped segment of its own over the arena's team; ``None`` when it cannot be set up
        (the outcome is the same on every rank of the team)."""
        from .symm import ArenaUnavailable, SymmetricArena

        try:
            return SymmetricArena(nbytes, self._team, self.device)
        except ArenaUnavailable:
            return None

    def _new_flat(self, arena, dtype: torch.dtype) -> torch.Tensor:
        if arena is not None:
            return arena.alloc(self.numel, dtype).zero_()
        return torch.zeros(self.numel, dtype=dtype, device=self.device)

    def release_grads(self) -> bool:
        """Free the gradient buffer (it holds no state between steps).  A slice of the job-wide arena
        cannot be freed: returns ``False`` and keeps it.  Collective over the team for a segment."""
        if self.grad_arena is not None and not self._own["grad"]:
            return False
        self.grad_data = torch.empty(0, dtype=self.grad_dtype, device=self.device)
        for p in self.params:
            p.main_grad = None
        if self.grad_arena is not None:
            self.grad_arena.close()
            self.grad_arena = None
        return True

    def restore_grads(self) -> None:
        if self.grad_data.numel():
            return
        if self._own["grad"]:
            self.grad_arena = self._segment(self.numel * self.grad_data.element_size() + 512)
        self.grad_data = self._new_flat(self.grad_arena, self.grad_dtype)
        self.rebind()

    def release_params(self, host: torch.Tensor) -> bool:
        """Copy the parameters to ``host`` (pinned) and free the device buffer.  Same rule as for the
        gradients: only a plain allocation or a segment of its own can go."""
        if self.param_arena is not None and not self._own["param"]:
            return False
        host.copy_(self.param_data, non_blocking=True)
        if self.device.type == "cuda":
            torch.cuda.current_stream().synchronize()
        self.param_data = torch.empty(0, dtype=self.param_dtype, device=self.device)
        for p in self.params:
            p.data = self.param_data
        if self.param_arena is not None:
            self.param_arena.close()
            self.param_arena = None
        return True

    def restore_params(self, host: torch.Tensor) -> None:
        if self.param_data.numel():
            return
        if self._own["param"]:
            self.param_arena = self._segment(self.numel * self.param_data.element_size() + 512)
        self.param_data = self._new_flat(self.param_arena, self.param_dtype)
        self.param_data.copy_(host, non_blocking=True)
        self.rebind()

    # ------------------------------------------------------------------------------------------
    def zero_grad(self) -> None:
        self.grad_data.zero_()

    def shard_range(self, dp_rank: Optional[int] = None) -> Tuple[int, int]:
        dp_rank = self.dp_rank if dp_rank is None else dp_rank
        per = self.numel // self.dp_size
        return dp_rank * per, (dp_rank + 1) * per

    def rebind(self) -> None:
        """Re-point parameters at the buffers (after the storage was released and re-created)."""
        for p, slot in zip(self.params, self.slots):
            p.data = self.param_data[slot.start:slot.start + slot.numel].view(slot.shape)
            p.main_grad = self.grad_data[slot.start:slot.start + slot.numel].view(slot.shape) \
                if self.grad_data is not None and self.grad_data.numel() else None

    # ---- buckets: contiguous ranges of whole parameters, in backward order ---------------------------
    def make_buckets(self, bucket_numel: int) -> List[Tuple[int, int]]:
        """Cut the buffer into ranges of at least ``bucket_numel`` elements that end on parameter
        boundaries, last parameters first (the order in which the backward finishes them)."""
        out: List[Tuple[int, int]] = []
        end = self.numel
        start = end
        for slot in reversed(self.slots):
            start = slot.start
            if end - start >= bucket_numel:
                out.append((start, end))
                end = start
        if end > 0:
            out.append((0, end))
        self.bucket_ranges = out
        self.bucket_of: Dict[int, int] = {}
        for pi, slot in enumerate(self.slots):
            for bi, (s0, e0) in enumerate(out):
                if s0 <= slot.start < e0:
                    self.bucket_of[pi] = bi
        return out

    def reduce_bucket(self, bi: int, group=None, average: bool = True, async_op: bool = False):
        """Reduce one bucket over the data-parallel group so that EVERY rank holds the reduced values of
        the range (a superset of what the distributed optimizer needs of it).  Peer-mapped buffers run
        the pull reduce-scatter and all-gather kernels on the range; otherwise one all-reduce, whose
        handle is returned when ``async_op``."""
        group = self.group if self.group is not None else group
        s0, e0 = self.bucket_ranges[bi]
        view = self.grad_data[s0:e0]
        scale = self.grad_scale if average else 1.0
        if self.dp_size == 1 or group is None:
            if self.is_expert and scale != 1.0:
                view.mul_(scale)
            return None
        if self.grad_arena is not None and (e0 - s0) % (8 * self.dp_size) == 0:
            ranks = self.grad_arena.team_ranks(group)
            per = (e0 - s0) // self.dp_size
            r = dist.get_rank(group)
            self.grad_arena.align(group)
            self.grad_arena.reduce_scatter(view, view[r * per:(r + 1) * per], scale=scale, ranks=ranks)
            self.grad_arena.all_gather_inplace(view, ranks=ranks)
            return None
        if scale != 1.0:
            view.mul_(scale)
        return dist.all_reduce(view, group=group, async_op=async_op)

    # ---- gradient reduction over the data-parallel group --------------------------------------------
    def reduce_grads(self, group=None, average: bool = True, to_shards: bool = False) -> None:
        """Sum (or average) gradients over DP.  ``to_shards=True`` leaves each rank with the
        reduced values of its own shard only (reduce-scatter, distributed optimizer)."""
        group = self.group if self.group is not None else group
        scale = self.grad_scale if average else 1.0
        if self.dp_size == 1 or group is None:
            if self.is_expert and scale != 1.0:   # experts without replicas still average over the DP tokens
                self.grad_data.mul_(scale)
            return
        if self.grad_arena is not None and to_shards:
            # one pull kernel: sum the peers' copies of my shard, scale, write my slice in place
            per = self.numel // self.dp_size
            r = dist.get_rank(group)
            # the ranks reach this point after unequal work (differently packed micro-batches):
            # a stream-ordered collective lines them up before the bounded device barrier
            self.grad_arena.align(group)
            self.grad_arena.reduce_scatter(self.grad_data, self.grad_data[r * per:(r + 1) * per],
                                           scale=scale, ranks=self.grad_arena.team_ranks(group))
            return
        if scale != 1.0:
            self.grad_data.mul_(scale)
        if to_shards:
            per = self.numel // self.dp_size
            r = dist.get_rank(group)
            out = self.grad_data[r * per:(r + 1) * per]
            dist.reduce_scatter_tensor(out, self.grad_data, group=group)
        else:
            dist.all_reduce(self.grad_data, group=group)

    def gather_params(self, group=None) -> None:
        """All-gather the parameter shards updated by the distributed optimizer."""
        group = self.group if self.group is not None else group
        if self.dp_size == 1 or group is None:
            return
        per = self.numel // self.dp_size
        r = dist.get_rank(group)
        if self.param_arena is not None:
            self.param_arena.all_gather_inplace(self.param_data, ranks=self.param_arena.team_ranks(group))
            return
        dist.all_gather_into_tensor(self.param_data, self.param_data[r * per:(r + 1) * per].clone(),
                                    group=group)


class ChunkedParamGather:
    """Parameter all-gather pipelined against the optimizer's update (``overlap_param_gather``; reference
    switch: ``mindspeed_rl/config_cls/megatron_config.py:353``).

    The distributed optimizer updates its contiguous shard chunk by chunk; as soon as chunk ``c`` is
    written on every rank, chunk ``c`` of every shard is fetched by all the others on a side stream
    (peer-mapped buffers: one copy-plan pull kernel between two device barriers; otherwise an
    asynchronous ``all_gather`` into the chunks' places), while the update of chunk ``c + 1`` runs.
    ``finish`` joins the side stream: when the optimizer step returns, every rank holds all parameters,
    exactly as after the plain one-shot all-gather."""

    def __init__(self, buf: "ParamAndGradBuffer", group, chunks: int = 8):
        self.buf, self.group = buf, buf.group if buf.group is not None else group
        self.world = buf.dp_size
        self.me = dist.get_rank(self.group)
        self.per = buf.numel // buf.dp_size
        esz = buf.param_data.element_size()
        unit = 16 // esz * 8                                   # chunk boundaries on 128-byte multiples
        n = max(1, min(chunks, self.per // unit))
        step = (self.per // n + unit - 1) // unit * unit
        self.bounds = [(lo, min(lo + step, self.per)) for lo in range(0, self.per, step)]
        self.side = torch.cuda.Stream() if buf.device.type == "cuda" else None
        self.handles: list = []
        self._plans: Dict[int, tuple] = {}

    def launch(self, c: int) -> None:
        """Chunk ``c`` of this rank's shard has been updated (on the current stream)."""
        buf, (lo, hi) = self.buf, self.bounds[c]
        arena = buf.param_arena
        if arena is not None:
            from .symm import plan_to_device

            if c not in self._plans:
                esz = buf.param_data.element_size()
                base = arena.offset_of(buf.param_data)
                ranks = arena.team_ranks(self.group)
                desc = [(ranks[r], base + (r * self.per + lo) * esz, (r * self.per + lo) * esz, 1, (hi - lo) * esz, 0, 0)
                        for r in range(self.world) if r != self.me]
                self._plans[c] = (plan_to_device(desc, buf.device), ranks)
            (plan, n_desc), ranks = self._plans[c]
            self.side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.side):
                arena.barrier(ranks)          # every member has written its chunk c
                arena.copy_plan(plan, n_desc, buf.param_data.view(torch.uint8), sync=False)
            return
        outs = [buf.param_data[r * self.per + lo:r * self.per + hi] for r in range(self.world)]
        mine = outs[self.me].clone()
        if self.side is not None:
            self.side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.side):
                dist.all_gather(outs, mine, group=self.group)
        else:
            self.handles.append(dist.all_gather(outs, mine, group=self.group, async_op=True))

    def finish(self) -> None:
        if self.side is not None:
            if self.buf.param_arena is not None:
                with torch.cuda.stream(self.side):
                    # nobody runs ahead into the next write of a chunk that a peer is still reading
                    self.buf.param_arena.barrier(self.buf.param_arena.team_ranks(self.group))
            torch.cuda.current_stream().wait_stream(self.side)
        for h in self.handles:
            h.wait()
        self.handles = []


def is_expert_param(name: str, p: nn.Parameter) -> bool:
    """Routed-expert weights: different on every expert-parallel rank (shared experts and the
    router are ordinary replicated parameters)."""
    return bool(getattr(p, "is_expert", False)) or ".experts." in f".{name}"


def expert_replica_groups(ps, cfg) -> dict:
    """Keyword arguments of :class:`DistributedDataParallel` that describe where the replicas of
    this rank's experts live (empty for dense models and without expert parallelism)."""
    if not getattr(cfg, "is_moe", False) or ps.size("ep") <= 1:
        return {}
    return dict(expert_dp_group=ps.group("edp"), expert_dp_size=ps.size("edp"), expert_dp_rank=ps.rank_in("edp"))


class DistributedDataParallel(nn.Module):
    """Wraps a model chunk, owns its :class:`ParamAndGradBuffer` and the DP group."""

    def __init__(self, module: nn.Module, dp_group=None, dp_size: int = 1,
                 grad_in_fp32: bool = False, bucket_numel: Optional[int] = None,
                 expert_dp_group=None, expert_dp_size: Optional[int] = None,
                 expert_dp_rank: Optional[int] = None, releasable_params: bool = False,
                 releasable_grads: bool = False, releasable_experts: bool = True, frozen_buffer: bool = False):
        """``expert_dp_*`` describe the ranks that hold replicas of this rank's experts (Megatron's
        expert-data-parallel group).  When given, the expert weights get a buffer of their own that
        is reduced, sharded (optimizer state) and gathered over that group only; without it
        every parameter is treated as replicated over ``dp_group``.

        ``releasable_params`` / ``releasable_grads``: on a machine with a peer-mapped arena give the flat
        parameter / gradient buffer a peer-mapped segment of its own, which the memory choreography of a
        co-located rollout can free and map again (``offload_train_param`` / ``offload_train_grad``);
        creating, freeing and re-creating a segment are collective over the arena's team, so every rank
        of the team must hold the same buffers (``releasable_experts=False`` leaves the expert buffer in
        the arena where pipeline stages differ in whether they have experts).  ``frozen_buffer``: also
        flatten the parameters that do not train (see ``frozen_buffer`` below)."""
        super().__init__()
        self.module = module
        self.dp_group, self.dp_size = dp_group, dp_size
        fp32_params = [(n, p) for n, p in module.named_parameters()
                       if p.requires_grad and p.dtype == torch.float32 and
                       next(module.parameters()).dtype != torch.float32]
        split_experts = expert_dp_size is not None and expert_dp_size != dp_size
        experts = [(n, p) for n, p in module.named_parameters()
                   if p.requires_grad and split_experts and is_expert_param(n, p)]
        taken = [q for _, q in fp32_params] + [q for _, q in experts]
        main = [(n, p) for n, p in module.named_parameters()
                if p.requires_grad and not any(p is q for q in taken)]
        self.buffers: List[ParamAndGradBuffer] = []
        gdt = torch.float32 if grad_in_fp32 else None
        if main:
            self.buffers.append(ParamAndGradBuffer(main, dp_size, gdt, bucket_numel, group=dp_group,
                                                   releasable_params=releasable_params,
                                                   releasable_grads=releasable_grads))
        if experts:
            self.buffers.append(ParamAndGradBuffer(
                experts, expert_dp_size, gdt, bucket_numel, group=expert_dp_group, dp_rank=expert_dp_rank,
                grad_scale=1.0 / max(dp_size, 1), is_expert=True,
                releasable_params=releasable_params and releasable_experts,
                releasable_grads=releasable_grads and releasable_experts))
        if fp32_params:  # e.g. the fp32 value head
            self.buffers.append(ParamAndGradBuffer(fp32_params, dp_size, torch.float32, bucket_numel,
                                                   group=dp_group))
        # frozen weights of a partly trainable model (base weights under LoRA): one parameter-only flat
        # buffer, outside ``buffers`` (no gradients, no optimizer state, nothing to reduce or gather)
        self.frozen_buffer: Optional[ParamAndGradBuffer] = None
        if frozen_buffer and main:
            dt = main[0][1].dtype
            frozen = [(n, p) for n, p in module.named_parameters() if not p.requires_grad and p.dtype == dt]
            if frozen:
                self.frozen_buffer = ParamAndGradBuffer(frozen, dp_size, None, bucket_numel, group=dp_group,
                                                        with_grads=False)

    def forward(self, *a, **kw):
        return self.module(*a, **kw)

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(self.module, name)

    def zero_grad_buffer(self) -> None:
        for b in self.buffers:
            b.zero_grad()

    # names of replicated parameters whose gradient is a partial sum over the TP ranks
    _TP_PARTIAL_ALWAYS = ("q_layernorm.weight", "k_layernorm.weight")          # each rank sees its own heads
    # norms and expert routers run on the local token shard (the value head runs on gathered tokens)
    _TP_PARTIAL_WITH_SP = ("input_layernorm.weight", "pre_mlp_layernorm.weight", "final_layernorm.weight",
                           "router.weight")

    def attach_tensor_parallel(self, tp_group, tp_size: int, sequence_parallel: bool) -> None:
        """Register the TP group so that ``finish_grad_sync`` can sum the gradients of replicated
        parameters that every TP rank computed from only its own heads / tokens (Megatron does
        the same for layer-norm gradients under sequence parallelism)."""
        self.tp_group, self.tp_size, self.tp_sequence_parallel = tp_group, tp_size, sequence_parallel

    def _tp_partial_grads(self) -> List[torch.Tensor]:
        pats = self._TP_PARTIAL_ALWAYS + (self._TP_PARTIAL_WITH_SP if getattr(self, "tp_sequence_parallel", False)
                                          else ())
        out = []
        for b in self.buffers:
            for p, slot in zip(b.params, b.slots):
                if getattr(p, "tp_reduce_grad", False) or slot.name.endswith(pats):
                    out.append(p.main_grad)
        return out

    # ---- gradient reduction overlapped with the backward (``overlap_grad_reduce``) ----------------------
    def enable_grad_overlap(self, bucket_numel: int = 40_000_000) -> None:
        """Cut the buffers into buckets of whole parameters.  While the last micro-batch of a step runs
        (``begin_last_microbatch``), the bucket of a layer is reduced over the data-parallel group as soon
        as the layer's backward has finished, on a side stream (CUDA) or as an asynchronous collective
        (CPU), while the backward of the earlier layers goes on; ``finish_grad_sync`` waits for those
        reductions and reduces what is left (embedding, head, final norm).  Reference switch:
        ``overlap_grad_reduce`` (``mindspeed_rl/config_cls/megatron_config.py:343``)."""
        self._home: Dict[int, Tuple[int, int]] = {}
        for bi, b in enumerate(self.buffers):
            b.make_buckets(bucket_numel)
            for pi, p in enumerate(b.params):
                self._home[id(p)] = (bi, pi)
        self.overlap_grad_reduce = True
        self._overlap = None

    def begin_last_microbatch(self) -> None:
        """Arm the overlapped reduction for the backward that follows (no-op unless enabled)."""
        if not getattr(self, "overlap_grad_reduce", False):
            return
        from ..models import gpt as _gpt

        pending = []
        for b in self.buffers:
            count = [0] * len(b.bucket_ranges)
            for pi in range(len(b.params)):
                count[b.bucket_of[pi]] += 1
            pending.append(count)
        cuda = self.buffers[0].device.type == "cuda"
        self._overlap = dict(pending=pending, launched=set(), handles=[],
                             side=(getattr(self, "_side_stream", None) or torch.cuda.Stream()) if cuda else None)
        if cuda:
            self._side_stream = self._overlap["side"]
        _gpt.grads_ready_hook[0] = self._layer_grads_ready

    def _layer_grads_ready(self, layer: nn.Module) -> None:
        st = self._overlap
        if st is None:
            return
        for p in layer.parameters():
            home = self._home.get(id(p))
            if home is None:
                continue
            bi, pi = home
            k = self.buffers[bi].bucket_of[pi]
            st["pending"][bi][k] -= 1
            if st["pending"][bi][k] == 0:
                self._launch_bucket(bi, k)

    def _launch_bucket(self, bi: int, k: int) -> None:
        st, b = self._overlap, self.buffers[bi]
        st["launched"].add((bi, k))
        if st["side"] is not None:
            st["side"].wait_stream(torch.cuda.current_stream())      # the bucket's gradients are complete
            with torch.cuda.stream(st["side"]):
                b.reduce_bucket(k, self.dp_group, average=True)
        else:
            h = b.reduce_bucket(k, self.dp_group, average=True, async_op=True)
            if h is not None:
                st["handles"].append(h)

    def _finish_overlap(self) -> bool:
        """Wait for the reductions started during the backward.  Returns True when the overlapped mode
        was armed (the caller then reduces only the buckets that were not launched)."""
        st = getattr(self, "_overlap", None)
        if st is None:
            return False
        from ..models import gpt as _gpt

        _gpt.grads_ready_hook[0] = None
        if st["side"] is not None:
            torch.cuda.current_stream().wait_stream(st["side"])
        for h in st["handles"]:
            h.wait()
        return True

    def finish_grad_sync(self, to_shards: bool = False) -> None:
        overlapped = self._finish_overlap()      # before anything else touches the gradient buffers
        if getattr(self, "tp_size", 1) > 1 and self.tp_group is not None:
            grads = self._tp_partial_grads()
            if grads:
                flat = torch.cat([g.reshape(-1).float() for g in grads])
                dist.all_reduce(flat, group=self.tp_group)
                off = 0
                for g in grads:
                    g.copy_(flat[off:off + g.numel()].view_as(g))
                    off += g.numel()
        if overlapped:
            st, self._overlap = self._overlap, None
            for bi, b in enumerate(self.buffers):
                for k in range(len(b.bucket_ranges)):
                    if (bi, k) not in st["launched"]:
                        b.reduce_bucket(k, self.dp_group, average=True)
            return
        for b in self.buffers:
            b.reduce_grads(self.dp_group, average=True, to_shards=to_shards)
