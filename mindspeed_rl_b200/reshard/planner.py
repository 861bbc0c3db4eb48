"""Train -> rollout weight resharding as a copy plan.

Training shards a model as ``TP_t x PP_t`` (x CP x DP); the rollout engine wants ``TP_i`` with the
whole depth on every rank (``PP_i = 1``) and more data-parallel replicas.  The reference walks
the parameters one by one: all-gather over train-TP, undo the fused QKV / gate-up interleaves,
broadcast over PP, re-split for the inference TP (``mindspeed_rl/workers/resharding/
vllm_weight_container.py:187-441``, ``weight_adaptor.py``).

Here the move is planned once on the host and executed by one kernel per reshard:

* every parameter is classified by how tensor parallelism cuts it (rows, GLU rows, columns,
  replicated / expert-local);
* for the rollout rank at hand, 1-D interval arithmetic yields for each destination tensor the
  list of source pieces ``(train rank, offset, pitch)`` -- TP shrink gathers pieces from several
  train ranks, TP growth takes a sub-range of one, PP gather takes each layer from the stage
  that owns it;
* the pieces become fixed-size descriptors executed by ``symm_copy_plan`` (direct peer reads from
  the peers' flat parameter buffers into the rollout buffer, over NVLink), or -- without a
  symmetric arena -- by ``execute_plan_torch`` over buffers gathered with ``torch.distributed``.

Fused-QKV needs no un-interleaving: the training layout groups ``[q.. k v]`` per KV group, a row
split by KV group is therefore a contiguous row range, and the rollout kernels read that layout
directly.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..models.transformer_config import TransformerConfig
from ..ops import QKVLayout
from ..parallel.state import ParallelState, RankLayout
from ..parallel.tp_comm import TPComm
from ..rollout.model_runner import LayerWeights, RolloutWeights

Desc = Tuple[int, int, int, int, int, int, int]   # src_rank, src_off, dst_off, rows, row_bytes, src_pitch, dst_pitch
_MAX_CHUNK = 64 << 20                              # contiguous copies are cut into pieces of this size


@dataclass
class Slot:
    start: int            # element offset inside the owning rank's flat parameter buffer
    shape: Tuple[int, ...]


def partition_kind(name: str) -> str:
    """How training tensor parallelism cuts a parameter."""
    if name.endswith(("linear_qkv.weight", "linear_qkv.bias", "word_embeddings.weight", "output_layer.weight")):
        return "rows"
    if name.endswith("linear_fc1.weight"):
        return "glu"
    if name.endswith(("linear_proj.weight", "linear_fc2.weight")):
        return "cols"
    return "local"


def intervals(n: int, n_src: int, n_dst: int, j: int) -> List[Tuple[int, int, int, int]]:
    """Cover destination shard ``j`` of ``n_dst`` equal shards of ``[0, n)`` with pieces of the
    ``n_src`` equal source shards: ``[(src_index, src_start, dst_start, length)]`` in local units."""
    if n % n_src or n % n_dst:
        raise ValueError(f"extent {n} is not divisible by the shard counts {n_src} / {n_dst}")
    ps, pd = n // n_src, n // n_dst
    lo, hi = j * pd, (j + 1) * pd
    out = []
    s = lo // ps
    while lo < hi:
        end = min(hi, (s + 1) * ps)
        out.append((s, lo - s * ps, lo - j * pd, end - lo))
        lo, s = end, s + 1
    return out


def _contig(src_rank: int, src_off: int, dst_off: int, nbytes: int) -> List[Desc]:
    out = []
    done = 0
    while done < nbytes:
        n = min(_MAX_CHUNK, nbytes - done)
        out.append((src_rank, src_off + done, dst_off + done, 1, n, 0, 0))
        done += n
    return out


def stage_layers(num_layers: int, pp: int, num_layer_list: Optional[Sequence[int]] = None) -> List[List[int]]:
    """Layers of every pipeline stage (no virtual stages, no empty slots)."""
    return [sum(chunks, []) for chunks in stage_chunks(num_layers, pp, num_layer_list)]


def pipeline_layout(mc, pp: int) -> List[List[List[int]]]:
    """``stage_chunks`` of a training config (``num_layers`` slots, ``num_layer_list``,
    ``num_layers_per_virtual_pipeline_stage``, ``noop_layers``)."""
    from ..models.transformer_config import parse_noop_layers

    per_virtual = getattr(mc, "num_layers_per_virtual_pipeline_stage", None)
    vpp = 1
    if per_virtual and pp > 1:
        if (mc.num_layers // pp) % per_virtual:
            raise ValueError("num_layers_per_virtual_pipeline_stage must divide the layer slots of a stage")
        vpp = mc.num_layers // pp // per_virtual
    return stage_chunks(mc.num_layers, pp, getattr(mc, "num_layer_list", None), vpp,
                        parse_noop_layers(getattr(mc, "noop_layers", None)))


def stage_chunks(num_layers: int, pp: int, num_layer_list: Optional[Sequence[int]] = None, vpp: int = 1,
                 noop_layers: Sequence[int] = ()) -> List[List[List[int]]]:
    """``[stage][chunk] -> layer numbers``.  ``num_layers`` counts layer SLOTS: with ``noop_layers``
    (slot indices that hold no layer, used to even out stages: reference flag ``noop_layers``,
    ``mindspeed_rl/config_cls/megatron_config.py:357``) the real layers are numbered consecutively
    in slot order.  Slots are dealt to virtual stages in order: virtual stage ``c * pp + s`` is
    chunk ``c`` of stage ``s`` (interleaved schedule, ``num_layers_per_virtual_pipeline_stage``);
    ``num_layer_list`` gives uneven slot counts per stage and excludes virtual stages."""
    vpp = max(int(vpp or 1), 1)
    if num_layer_list:
        if vpp > 1:
            raise ValueError("num_layer_list and a virtual pipeline cannot be combined")
        counts = list(num_layer_list)
    else:
        if num_layers % (pp * vpp):
            raise ValueError(f"{num_layers} layer slots do not divide into {pp} x {vpp} (virtual) stages")
        counts = [num_layers // (pp * vpp)] * (pp * vpp)
    if sum(counts) != num_layers:
        raise ValueError("pipeline layer counts do not add up to num_layers")
    noop = set(int(i) for i in (noop_layers or ()))
    real, nxt = {}, 0
    for slot in range(num_layers):
        if slot not in noop:
            real[slot] = nxt
            nxt += 1
    out: List[List[List[int]]] = [[] for _ in range(pp)]
    s = 0
    for v, c in enumerate(counts):
        out[v % pp].append([real[i] for i in range(s, s + c) if i in real])
        s += c
    return out


@dataclass
class ReshardPlan:
    desc: List[Desc]
    tensors: Dict[str, Tuple[int, Tuple[int, ...]]]   # global name -> (byte offset in dst, shape)
    nbytes: int


def build_plan(cfg: TransformerConfig, train: RankLayout, infer_tp: int, rank: int,
               stage_slots: Sequence[Dict[str, Slot]], layers_of_stage: Sequence[Sequence[int]],
               src_base: Callable[[int], int], esz: int = 2) -> ReshardPlan:
    """Plan for global rank ``rank``.

    ``stage_slots[s]`` maps the state-dict names of pipeline stage ``s`` (local layer indices) to
    their slots; ``src_base(r)`` is the byte address offset of rank ``r``'s parameter buffer
    (arena offset, or 0 when the sources are separate gathered buffers).  Destination names use
    *global* layer indices.
    """
    tp_t = train.tp
    coords = train.coords(rank)
    j = rank % infer_tp                                   # rollout TP rank (TP is the fastest dim)

    def src_rank(tp_idx: int, stage: int) -> int:
        return train.rank_of(tp=tp_idx, pp=stage, dp=coords["dp"], cp=coords["cp"])

    desc: List[Desc] = []
    tensors: Dict[str, Tuple[int, Tuple[int, ...]]] = {}
    cursor = 0

    def place(name: str, shape: Tuple[int, ...]) -> int:
        nonlocal cursor
        off = (cursor + 255) // 256 * 256
        n = esz
        for d in shape:
            n *= d
        cursor = off + n
        tensors[name] = (off, tuple(shape))
        return off

    def emit(gname: str, lname: str, stage: int) -> None:
        slot = stage_slots[stage][lname]
        kind = partition_kind(lname)
        shape = tuple(slot.shape)
        inner = esz
        for d in shape[1:]:
            inner *= d                                    # bytes of one dim-0 row
        if kind == "local" or tp_t == infer_tp:
            # replicated / expert-local tensors and unchanged TP: take this rank's own TP index
            r = src_rank(coords["tp"] if kind == "local" else j, stage)
            dst = place(gname, shape)
            desc.extend(_contig(r, src_base(r) + slot.start * esz, dst, shape[0] * inner if shape else esz))
            return
        if kind == "rows":
            full = shape[0] * tp_t
            dshape = (full // infer_tp,) + shape[1:]
            dst = place(gname, dshape)
            for s, s0, d0, ln in intervals(full, tp_t, infer_tp, j):
                r = src_rank(s, stage)
                desc.extend(_contig(r, src_base(r) + slot.start * esz + s0 * inner, dst + d0 * inner, ln * inner))
        elif kind == "glu":
            half_t = shape[0] // 2
            full = half_t * tp_t
            half_i = full // infer_tp
            dshape = (2 * half_i,) + shape[1:]
            dst = place(gname, dshape)
            for blk in (0, 1):                            # gate rows, then up rows
                for s, s0, d0, ln in intervals(full, tp_t, infer_tp, j):
                    r = src_rank(s, stage)
                    desc.extend(_contig(r, src_base(r) + slot.start * esz + (blk * half_t + s0) * inner,
                                        dst + (blk * half_i + d0) * inner, ln * inner))
        elif kind == "cols":
            rows, k_t = shape[0], shape[1]
            full = k_t * tp_t
            k_i = full // infer_tp
            dst = place(gname, (rows, k_i))
            for s, s0, d0, ln in intervals(full, tp_t, infer_tp, j):
                r = src_rank(s, stage)
                desc.append((r, src_base(r) + slot.start * esz + s0 * esz, dst + d0 * esz, rows, ln * esz,
                             k_t * esz, k_i * esz))
        else:
            raise ValueError(kind)

    for stage, layer_ids in enumerate(layers_of_stage):
        table = stage_slots[stage]
        if "embedding.word_embeddings.weight" in table:
            emit("embedding.word_embeddings.weight", "embedding.word_embeddings.weight", stage)
        for local, layer in enumerate(layer_ids):
            prefix = f"decoder.layers.{local}."
            for lname in table:
                if lname.startswith(prefix):
                    emit(f"decoder.layers.{layer}." + lname[len(prefix):], lname, stage)
        for lname in ("decoder.final_layernorm.weight", "output_layer.weight"):
            if lname in table:
                emit(lname, lname, stage)
    return ReshardPlan(desc, tensors, (cursor + 255) // 256 * 256)


def execute_plan_torch(plan: ReshardPlan, sources: Dict[int, torch.Tensor], dst: torch.Tensor) -> None:
    """Reference executor: ``sources[r]`` is rank r's parameter buffer viewed as bytes (uint8),
    ``dst`` the destination bytes.  Used on CPU and as the oracle of the copy-plan kernel."""
    for src_rank, src_off, dst_off, rows, row_bytes, sp, dp in plan.desc:
        s = sources[src_rank]
        if rows == 1:
            dst[dst_off:dst_off + row_bytes] = s[src_off:src_off + row_bytes]
        else:
            sv = torch.as_strided(s, (rows, row_bytes), (sp, 1), src_off)
            torch.as_strided(dst, (rows, row_bytes), (dp, 1), dst_off).copy_(sv)


def weights_from_buffer(cfg: TransformerConfig, infer_tp: int, tp_rank: int, plan: ReshardPlan,
                        buf: torch.Tensor, dtype: torch.dtype, moe_builder: Optional[Callable] = None
                        ) -> RolloutWeights:
    """Views into the destination buffer (bytes) arranged as the rollout model runner wants them."""
    def t(name: str) -> Optional[torch.Tensor]:
        if name not in plan.tensors:
            return None
        off, shape = plan.tensors[name]
        n = 1
        for d in shape:
            n *= d
        return buf[off:off + n * buf.new_empty(0, dtype=dtype).element_size()].view(dtype).view(shape)

    layers = []
    for li in range(cfg.num_layers):
        p = f"decoder.layers.{li}."
        kw = dict(input_norm=t(p + "input_layernorm.weight"), qkv_w=t(p + "self_attention.linear_qkv.weight"),
                  qkv_b=t(p + "self_attention.linear_qkv.bias"), o_w=t(p + "self_attention.linear_proj.weight"),
                  post_norm=t(p + "pre_mlp_layernorm.weight"), q_norm=t(p + "self_attention.q_layernorm.weight"),
                  k_norm=t(p + "self_attention.k_layernorm.weight"))
        if p + "mlp.linear_fc1.weight" in plan.tensors:
            kw.update(gate_up_w=t(p + "mlp.linear_fc1.weight"), down_w=t(p + "mlp.linear_fc2.weight"))
        elif moe_builder is not None:
            kw.update(moe=moe_builder(li, t))
        else:
            raise NotImplementedError("expert layers need a moe_builder")
        layers.append(LayerWeights(**kw))
    head = t("output_layer.weight")
    embed = t("embedding.word_embeddings.weight")
    layout = QKVLayout(cfg.num_attention_heads // infer_tp, cfg.num_query_groups // infer_tp, cfg.head_dim,
                       interleaved=True)
    return RolloutWeights(embed=embed, layers=layers, final_norm=t("decoder.final_layernorm.weight"),
                          lm_head=head if head is not None else embed, qkv_layout=layout,
                          vocab_start=tp_rank * (cfg.vocab_size // infer_tp))


DECODE_ALL_REDUCE_TOKENS = 1024     # largest token count whose hidden states go through the peer-memory all-reduce


def attach_peer_all_reduce(comm: TPComm, arena, hidden_size: int) -> None:
    """Give the rollout's TP communicator the peer-memory all-reduce for decode-sized messages
    (``MSRL_PEER_ALLREDUCE=0`` keeps the library collective).  Collective over the arena's team: every
    rank of the job calls it at the same point."""
    import os

    if arena is None or comm.world_size <= 1 or comm.group is None or os.environ.get("MSRL_PEER_ALLREDUCE", "1") != "1":
        return
    if comm.world_size > 2 and os.environ.get("MSRL_PEER_ALLREDUCE_WIDE", "0") != "1":
        return     # pushing to three or more peers multiplies the bytes sent: measured slower than the library there
    need = DECODE_ALL_REDUCE_TOKENS * hidden_size * 2
    if arena.free_bytes() < 2 * comm.world_size * need + (1 << 20):
        return
    comm.peer_ar = arena.make_all_reduce(need, arena.team_ranks(comm.group))


class Resharder:
    """Owns the rollout-side parallel state, engine and weight buffer of one worker."""

    def __init__(self, cfg: TransformerConfig, ddp, train_state: ParallelState, infer_tp: int, device,
                 engine_factory: Callable, arena=None, num_layer_list: Optional[Sequence[int]] = None,
                 layers_of_stage: Optional[Sequence[Sequence[int]]] = None):
        self.cfg, self.ddp, self.train_state, self.infer_tp = cfg, ddp, train_state, infer_tp
        self.device = torch.device(device)
        self.arena = arena
        layout = train_state.layout
        if layout.world_size % infer_tp:
            raise ValueError("the rollout TP size must divide the world size")
        if cfg.is_moe and layout.ep > 1 and (layout.pp > 1 or getattr(layout, "expert_tp", 1) > 1):
            raise NotImplementedError("with expert parallelism the experts stay on their training ranks: only the "
                                      "dense tensors are resharded, which needs pp = 1 and unsplit experts")
        self.infer_state = ParallelState(RankLayout(layout.world_size, tp=infer_tp), train_state.rank,
                                         backend=train_state.backend, rank_offset=train_state.rank_offset)
        tp_group = self.infer_state.group("tp")
        self.comm = TPComm(tp_group, False, world_size=infer_tp, rank=self.infer_state.rank_in("tp"))
        attach_peer_all_reduce(self.comm, arena, cfg.hidden_size)
        self.infer_cfg = dataclasses.replace(cfg, tensor_model_parallel_size=infer_tp, sequence_parallel=False)
        self.engine = engine_factory(self.infer_cfg, self.comm if infer_tp > 1 else None)
        self.buffer: Optional[torch.Tensor] = None
        self._plan: Optional[ReshardPlan] = None
        self._plan_dev = None
        self._layers = [list(l) for l in layers_of_stage] if layers_of_stage is not None else \
            stage_layers(cfg.num_layers, layout.pp, num_layer_list)
        self.last_bytes = 0

    @classmethod
    def for_worker(cls, worker, gc) -> "Resharder":
        from ..parallel.symm import get_arena
        from ..rollout.engine import LLMEngine

        def factory(icfg, comm):
            return LLMEngine(icfg, worker.device, max_num_seqs=gc.max_num_seqs,
                             max_num_batched_tokens=gc.max_num_batched_tokens, max_model_len=gc.max_model_len,
                             block_size=gc.kv_block_size, enable_prefix_caching=gc.enable_prefix_caching,
                             enforce_eager=gc.enforce_eager, graph_batch_sizes=tuple(gc.graph_batch_sizes),
                             eos_token_id=worker.eos_token_id, pad_token_id=worker.pad_token_id, comm=comm,
                             seed=worker.seed,
                             lockstep_group=worker.parallel_state.group("ep")
                             if (worker.tcfg.is_moe and worker.parallel_state.size("ep") > 1) else None)

        return cls(worker.tcfg, worker.model, worker.parallel_state, gc.infer_tensor_parallel_size, worker.device,
                   factory, arena=get_arena(),
                   layers_of_stage=[sum(ch, []) for ch in
                                    pipeline_layout(worker.actor_config, worker.parallel_state.size("pp"))])

    # ------------------------------------------------------------------------------------------
    def _main_buffer(self):
        return self.ddp.buffers[0]

    def _param_arena(self):
        """The peer-mapped home of the training parameters (the job-wide arena or the buffer's own
        segment), or ``None`` when they are a plain allocation."""
        return getattr(self._main_buffer(), "param_arena", None) if self.arena is not None else None

    def _use_arena(self) -> bool:
        return self._param_arena() is not None

    def _build(self) -> None:
        ps = self.train_state
        buf = self._main_buffer()
        mine = {s.name: Slot(s.start, tuple(s.shape)) for s in buf.slots}
        base = self._param_arena().offset_of(buf.param_data) if self._use_arena() else 0
        stage = ps.rank_in("pp")
        info = (ps.rank, stage, base, mine if ps.rank_in("tp") == 0 else None)
        if dist.is_initialized() and ps.size("mp") > 1:
            box: List = [None] * ps.size("mp")
            dist.all_gather_object(box, info, group=ps.group("mp"))
        else:
            box = [info]
        tables: List[Optional[Dict[str, Slot]]] = [None] * ps.size("pp")
        bases: Dict[int, int] = {}
        for r, st, b, table in box:
            bases[r] = b
            if table is not None:
                tables[st] = table
        if self._use_arena():
            # arena ranks are positions in the arena's team; the team is the whole job here
            src_base = lambda r: bases[r]
        else:
            src_base = lambda r: 0
        esz = buf.param_data.element_size()
        self._plan = build_plan(self.cfg, ps.layout, self.infer_tp, ps.rank, tables, self._layers, src_base, esz)
        if self._use_arena():
            from ..parallel.symm import plan_to_device

            self._plan_dev = plan_to_device(self._plan.desc, self.device)

    def _moe_builder(self, core):
        def build(li, t):
            return core.decoder.layers[li].mlp.rollout_view()
        return build

    @torch.no_grad()
    def reshard(self, core) -> RolloutWeights:
        if self._plan is None:
            self._build()
        plan = self._plan
        buf = self._main_buffer()
        if self.buffer is None:
            self.buffer = torch.empty(plan.nbytes, dtype=torch.uint8, device=self.device)
        timed = self.device.type == "cuda"
        if timed:
            # device time of the move itself (entry barrier + copy-plan kernel + exit barrier); the
            # events are read by ``device_ms`` after the caller's next synchronisation
            self._events = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            self._events[0].record()
        if self._use_arena():
            # the ranks arrive from the update stage at different times: line them up before the
            # bounded device barrier (outside the timed interval: it is waiting, not resharding)
            home = self._param_arena()
            home.align()
            if timed:
                self._events[0].record()
            home.copy_plan(self._plan_dev[0], self._plan_dev[1], self.buffer, sync=True)
        else:
            self._gathered_copy(plan, buf)
        if timed:
            self._events[1].record()
        self.last_bytes = sum(d[3] * d[4] for d in plan.desc)
        return weights_from_buffer(self.infer_cfg, self.infer_tp, self.infer_state.rank_in("tp"), plan, self.buffer,
                                   buf.param_dtype, self._moe_builder(core) if self.cfg.is_moe else None)

    def _gathered_copy(self, plan: ReshardPlan, buf) -> None:
        """Library fallback: all-gather the parameter buffers of the model-parallel group, then
        run the plan locally."""
        ps = self.train_state
        local = buf.param_data.view(torch.uint8)
        if dist.is_initialized() and ps.size("mp") > 1:
            sizes = [None] * ps.size("mp")
            dist.all_gather_object(sizes, int(local.numel()), group=ps.group("mp"))
            cap = max(sizes)
            padded = torch.zeros(cap, dtype=torch.uint8, device=local.device)
            padded[:local.numel()] = local
            got = [torch.empty_like(padded) for _ in sizes]
            dist.all_gather(got, padded, group=ps.group("mp"))
            sources = {r: g for r, g in zip(ps.ranks("mp"), got)}
        else:
            sources = {ps.rank: local}
        execute_plan_torch(plan, sources, self.buffer)

    def device_ms(self) -> Optional[float]:
        """Device time of the last :meth:`reshard` in milliseconds (synchronises on its end event)."""
        ev = getattr(self, "_events", None)
        if ev is None:
            return None
        ev[1].synchronize()
        return float(ev[0].elapsed_time(ev[1]))

    def release(self) -> None:
        self.buffer = None
