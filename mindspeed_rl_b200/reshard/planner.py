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

Routed experts move through the same plan when the rollout's expert layout differs from training
(``ExpertPlacement``): a rollout rank lists the logical experts it hosts (its share of an
``infer_expert_parallel_size``-way split, or the entry of an expert-load-balancing map, which may
host an expert on several ranks) and the plan pulls each expert's ``[gate | up]`` column block and
its down-projection rows from the training rank that owns it (reference: EP -> TP conversion, EP
growth, expert send / receive and redundant experts in ``vllm_weight_container.py:226-266,336-420,
487-588``).  Low-rank adapters travel as ordinary tensors (``B`` cut like the weight's output rows,
``A`` like its input columns) and are folded into the rollout copy of the weights after the copy,
``W += (alpha / r) B A``, so the rollout never sees an adapter.
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
    buf: int = 0          # which of the rank's flat buffers (0: trainable dense, then experts, frozen, fp32)
    esz: int = 0          # bytes per element (0: the plan's default), e.g. 4 for an fp32 router in a bf16 model


@dataclass
class ExpertPlacement:
    """Where the routed experts of the rollout come from."""
    e_local_train: int                          # experts per training expert-parallel rank
    hosted: Callable[[int], Sequence[int]]      # global layer number -> logical expert ids this rollout rank hosts
    src_rank: Callable[[int, int], int]         # (training expert-parallel index, pipeline stage) -> global rank


def partition_kind(name: str) -> str:
    """How training tensor parallelism cuts a parameter."""
    if name.endswith(("linear_qkv.weight", "linear_qkv.bias", "word_embeddings.weight", "output_layer.weight",
                      "linear_qkv.lora_B",
                      # latent attention: the up-projections hold whole heads, head-major
                      "linear_q_up_proj.weight", "linear_kv_up_proj.weight", "linear_q_proj.weight")):
        return "rows"
    if name.endswith(("linear_fc1.weight", "linear_fc1.lora_B")):
        return "glu"
    if name.endswith(("linear_proj.weight", "linear_fc2.weight", "linear_proj.lora_A", "linear_fc2.lora_A")):
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
    desc_buf: Optional[List[int]] = None              # source buffer index of every descriptor (None: all 0)
    esz_of: Optional[Dict[str, int]] = None           # element size of tensors that differ from the plan's default

    def buf_of(self, i: int) -> int:
        return self.desc_buf[i] if self.desc_buf is not None else 0


def build_plan(cfg: TransformerConfig, train: RankLayout, infer_tp: int, rank: int,
               stage_slots: Sequence[Dict[str, Slot]], layers_of_stage: Sequence[Sequence[int]],
               src_base: Callable[..., int], esz: int = 2,
               experts: Optional[ExpertPlacement] = None) -> ReshardPlan:
    """Plan for global rank ``rank``.

    ``stage_slots[s]`` maps the state-dict names of pipeline stage ``s`` (local layer indices) to
    their slots; ``src_base(r, buf)`` is the byte address offset of flat buffer ``buf`` of rank ``r``
    (arena offset, or 0 when the sources are separate gathered buffers; a one-argument callable is
    taken to ignore ``buf``).  Destination names use *global* layer indices.  ``experts``: re-home the
    routed experts (otherwise expert tensors are copied as they are on this rank).
    """
    import inspect

    if len(inspect.signature(src_base).parameters) == 1:
        _one = src_base
        src_base = lambda r, b=0: _one(r)
    tp_t = train.tp
    coords = train.coords(rank)
    j = rank % infer_tp                                   # rollout TP rank (TP is the fastest dim)

    def src_rank(tp_idx: int, stage: int) -> int:
        return train.rank_of(tp=tp_idx, pp=stage, dp=coords["dp"], cp=coords["cp"])

    desc: List[Desc] = []
    desc_buf: List[int] = []
    tensors: Dict[str, Tuple[int, Tuple[int, ...]]] = {}
    cursor = 0

    def add(items: List[Desc], buf: int) -> None:
        desc.extend(items)
        desc_buf.extend([buf] * len(items))

    esz_of: Dict[str, int] = {}
    default_esz = esz

    def place(name: str, shape: Tuple[int, ...]) -> int:
        nonlocal cursor
        off = (cursor + 255) // 256 * 256
        n = esz
        for d in shape:
            n *= d
        cursor = off + n
        tensors[name] = (off, tuple(shape))
        if esz != default_esz:
            esz_of[name] = esz
        return off

    def emit(gname: str, lname: str, stage: int) -> None:
        nonlocal esz
        slot = stage_slots[stage][lname]
        esz = slot.esz or default_esz
        kind = partition_kind(lname)
        shape = tuple(slot.shape)
        inner = esz
        for d in shape[1:]:
            inner *= d                                    # bytes of one dim-0 row
        if kind == "local" or tp_t == infer_tp:
            # replicated / expert-local tensors and unchanged TP: take this rank's own TP index
            r = src_rank(coords["tp"] if kind == "local" else j, stage)
            dst = place(gname, shape)
            add(_contig(r, src_base(r, slot.buf) + slot.start * esz, dst, shape[0] * inner if shape else esz), slot.buf)
            return
        if kind == "rows":
            full = shape[0] * tp_t
            dshape = (full // infer_tp,) + shape[1:]
            dst = place(gname, dshape)
            for s, s0, d0, ln in intervals(full, tp_t, infer_tp, j):
                r = src_rank(s, stage)
                add(_contig(r, src_base(r, slot.buf) + slot.start * esz + s0 * inner, dst + d0 * inner, ln * inner),
                    slot.buf)
        elif kind == "glu":
            half_t = shape[0] // 2
            full = half_t * tp_t
            half_i = full // infer_tp
            dshape = (2 * half_i,) + shape[1:]
            dst = place(gname, dshape)
            for blk in (0, 1):                            # gate rows, then up rows
                for s, s0, d0, ln in intervals(full, tp_t, infer_tp, j):
                    r = src_rank(s, stage)
                    add(_contig(r, src_base(r, slot.buf) + slot.start * esz + (blk * half_t + s0) * inner,
                                dst + (blk * half_i + d0) * inner, ln * inner), slot.buf)
        elif kind == "cols":
            rows, k_t = shape[0], shape[1]
            full = k_t * tp_t
            k_i = full // infer_tp
            dst = place(gname, (rows, k_i))
            for s, s0, d0, ln in intervals(full, tp_t, infer_tp, j):
                r = src_rank(s, stage)
                add([(r, src_base(r, slot.buf) + slot.start * esz + s0 * esz, dst + d0 * esz, rows, ln * esz,
                      k_t * esz, k_i * esz)], slot.buf)
        else:
            raise ValueError(kind)

    def emit_experts(gname: str, lname: str, stage: int, layer: int) -> None:
        """Gather the hosted experts of ``layer`` from their training owners into rollout slot order."""
        nonlocal esz
        slot = stage_slots[stage][lname]
        esz = slot.esz or default_esz
        ids = list(experts.hosted(layer))
        e_t, n_loc = experts.e_local_train, len(ids)
        if lname.endswith("experts.weight1"):                # [H, E_local * 2F]: one column block per expert
            h, cols = slot.shape
            w = cols // e_t
            dst = place(gname, (h, n_loc * w))
            for q, e in enumerate(ids):
                r = experts.src_rank(e // e_t, stage)
                add([(r, src_base(r, slot.buf) + (slot.start + (e % e_t) * w) * esz, dst + q * w * esz, h, w * esz,
                      cols * esz, n_loc * w * esz)], slot.buf)
        else:                                                # [E_local * F, H]: one block of rows per expert
            rows, h = slot.shape
            f = rows // e_t
            dst = place(gname, (n_loc * f, h))
            for q, e in enumerate(ids):
                r = experts.src_rank(e // e_t, stage)
                add(_contig(r, src_base(r, slot.buf) + (slot.start + (e % e_t) * f * h) * esz, dst + q * f * h * esz,
                            f * h * esz), slot.buf)

    for stage, layer_ids in enumerate(layers_of_stage):
        table = stage_slots[stage]
        if "embedding.word_embeddings.weight" in table:
            emit("embedding.word_embeddings.weight", "embedding.word_embeddings.weight", stage)
        for local, layer in enumerate(layer_ids):
            prefix = f"decoder.layers.{local}."
            for lname in table:
                if not lname.startswith(prefix):
                    continue
                gname = f"decoder.layers.{layer}." + lname[len(prefix):]
                if experts is not None and lname.endswith(("experts.weight1", "experts.weight2")):
                    emit_experts(gname, lname, stage, layer)
                else:
                    emit(gname, lname, stage)
        for lname in ("decoder.final_layernorm.weight", "output_layer.weight"):
            if lname in table:
                emit(lname, lname, stage)
    return ReshardPlan(desc, tensors, (cursor + 255) // 256 * 256, desc_buf if any(desc_buf) else None,
                       esz_of or None)


def execute_plan_torch(plan: ReshardPlan, sources: Dict[int, torch.Tensor], dst: torch.Tensor) -> None:
    """Reference executor: ``sources[r]`` is rank r's parameter buffer viewed as bytes (uint8),
    ``dst`` the destination bytes.  Used on CPU and as the oracle of the copy-plan kernel."""
    for i, (src_rank, src_off, dst_off, rows, row_bytes, sp, dp) in enumerate(plan.desc):
        b = plan.buf_of(i)
        s = sources[(src_rank, b)] if (src_rank, b) in sources else sources[src_rank]
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
        dt = dtype
        if plan.esz_of and name in plan.esz_of:
            dt = {4: torch.float32, 2: torch.bfloat16 if dtype != torch.float16 else torch.float16}[plan.esz_of[name]]
        return buf[off:off + n * buf.new_empty(0, dtype=dt).element_size()].view(dt).view(shape)

    def fold(prefix: str) -> None:
        """``W += (alpha / r) B A`` on the rollout copy of an adapted linear (fp32 sum, one rounding)."""
        a, b, w = t(prefix + ".lora_A"), t(prefix + ".lora_B"), t(prefix + ".weight")
        if a is None or b is None or w is None:
            return
        scale = float(cfg.lora_alpha) / float(cfg.lora_r)
        w.copy_((w.float() + scale * torch.matmul(b.float(), a.float())).to(w.dtype))

    layers = []
    for li in range(cfg.num_layers):
        p = f"decoder.layers.{li}."
        if getattr(cfg, "lora_r", 0):
            for holder in ("self_attention.linear_qkv", "self_attention.linear_proj", "mlp.linear_fc1", "mlp.linear_fc2"):
                fold(p + holder)
        if getattr(cfg, "multi_latent_attention", False):
            from ..models.mla import MLASelfAttention

            sa = p + "self_attention."
            names = [n[len(sa):] for n in plan.tensors if n.startswith(sa)]
            block = MLASelfAttention.from_tensors(cfg, infer_tp, {n: t(sa + n) for n in names})
            if not block.rollout_supported():
                raise NotImplementedError(
                    "rollout of latent attention needs query/key and value heads of one common size 64 or 128 "
                    f"(got {block.qd} / {block.vd}): the paged KV cache stores full per-head keys and values")
            kw = dict(input_norm=t(p + "input_layernorm.weight"), qkv_w=None, qkv_b=None, mla=block,
                      o_w=t(sa + "linear_proj.weight"), post_norm=t(p + "pre_mlp_layernorm.weight"))
        else:
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
    if getattr(cfg, "multi_latent_attention", False):
        nh = cfg.num_attention_heads // infer_tp           # one key / value head per query head, full size
        layout = QKVLayout(nh, nh, cfg.qk_head_dim + cfg.qk_pos_emb_head_dim, interleaved=True)
    else:
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


def wanted_infer_ep(cfg: TransformerConfig, layout: RankLayout, gc) -> Optional[int]:
    """Expert-parallel size of the rollout asked for by the generation config, or ``None`` when the
    experts can stay where training has them (dense model, same size, nothing configured)."""
    if not cfg.is_moe:
        return None
    want = getattr(gc, "infer_expert_parallel_size", None)
    if not want or int(want) == layout.ep_total:
        return None
    return int(want)


class Resharder:
    """Owns the rollout-side parallel state, engine and weight buffer of one worker."""

    def __init__(self, cfg: TransformerConfig, ddp, train_state: ParallelState, infer_tp: int, device,
                 engine_factory: Callable, arena=None, num_layer_list: Optional[Sequence[int]] = None,
                 layers_of_stage: Optional[Sequence[Sequence[int]]] = None, infer_ep: Optional[int] = None,
                 expert_map: Optional[dict] = None):
        """``infer_ep``: expert-parallel size of the rollout (``None``: the experts stay where training has
        them); ``expert_map``: placement produced by the expert-load balancer (``rollout.eplb.
        expert_map_from_counts``: per MoE layer and rollout expert-parallel rank the logical experts it
        hosts, possibly with replicas)."""
        self.cfg, self.ddp, self.train_state, self.infer_tp = cfg, ddp, train_state, infer_tp
        self.device = torch.device(device)
        self.arena = arena
        layout = train_state.layout
        if layout.world_size % infer_tp:
            raise ValueError("the rollout TP size must divide the world size")
        self.expert_map = expert_map
        self.infer_ep = layout.ep_total if (infer_ep is None or not cfg.is_moe) else int(infer_ep)
        # the experts move when the rollout wants another expert layout than training has
        self.rehome = bool(cfg.is_moe and (self.infer_ep != layout.ep_total or expert_map is not None
                                           or (layout.pp > 1 and layout.ep_total > 1)))
        if cfg.is_moe and layout.ep_total > 1 and layout.expert_tp > 1:
            raise NotImplementedError("experts that training splits over tensor-parallel ranks cannot be resharded; "
                                      "use moe_tp_extend_ep or tensor_model_parallel_size = 1 for expert models")
        if self.rehome and layout.pp > 1 and getattr(cfg, "moe_router_enable_expert_bias", False):
            raise NotImplementedError("the routers' selection bias lives on the stage that owns the layer: re-homing "
                                      "experts across pipeline stages is not supported with aux-loss-free balancing")
        if self.rehome:
            n_phys = self._physical_experts()
            if n_phys % self.infer_ep or layout.world_size % (infer_tp * self.infer_ep):
                raise ValueError(f"{n_phys} rollout expert slots / {layout.world_size} ranks do not divide into "
                                 f"tp {infer_tp} x ep {self.infer_ep}")
            self.infer_state = ParallelState(RankLayout(layout.world_size, tp=infer_tp, ep=self.infer_ep),
                                             train_state.rank, backend=train_state.backend,
                                             rank_offset=train_state.rank_offset)
        else:
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

        expert_map = None
        if worker.tcfg.is_moe and getattr(gc, "expert_map_path", None):
            import json

            with open(gc.expert_map_path) as fh:
                expert_map = json.load(fh)
        infer_ep = wanted_infer_ep(worker.tcfg, worker.parallel_state.layout, gc)
        holder = {}

        def factory(icfg, comm):
            # the engines of one rollout expert-parallel group exchange tokens in every forward: they
            # step together (the group is known once the rollout state exists)
            return LLMEngine(icfg, worker.device, max_num_seqs=gc.max_num_seqs,
                             max_num_batched_tokens=gc.max_num_batched_tokens, max_model_len=gc.max_model_len,
                             block_size=gc.kv_block_size, enable_prefix_caching=gc.enable_prefix_caching,
                             enforce_eager=gc.enforce_eager, graph_batch_sizes=tuple(gc.graph_batch_sizes),
                             eos_token_id=worker.eos_token_id, pad_token_id=worker.pad_token_id, comm=comm,
                             seed=worker.seed, lockstep_group=holder["self"]._lockstep_group())

        self = cls.__new__(cls)
        holder["self"] = self
        self.__init__(worker.tcfg, worker.model, worker.parallel_state, gc.infer_tensor_parallel_size, worker.device,
                      factory, arena=get_arena(),
                      layers_of_stage=[sum(ch, []) for ch in
                                       pipeline_layout(worker.actor_config, worker.parallel_state.size("pp"))],
                      infer_ep=infer_ep, expert_map=expert_map)
        return self

    def _lockstep_group(self):
        if not self.cfg.is_moe:
            return None
        if self.rehome:
            return self.infer_state.group("ep") if self.infer_ep > 1 else None
        return self.train_state.group("ep") if self.train_state.size("ep") > 1 else None

    # ---- expert placement ------------------------------------------------------------------------
    def _physical_experts(self) -> int:
        """Expert slots of the rollout over all its expert-parallel ranks (logical experts + replicas)."""
        if self.expert_map is None:
            return self.cfg.num_experts
        first = self.expert_map["layer_list"][0]
        if first["device_count"] != self.infer_ep:
            raise ValueError(f"the expert map places experts on {first['device_count']} devices, the rollout has "
                             f"{self.infer_ep} expert-parallel ranks")
        return sum(len(d["device_expert"]) for d in first["device_list"])

    def _moe_index(self, layer: int) -> int:
        return sum(1 for i in range(layer) if self.cfg.layer_is_moe(i))

    def hosted_experts(self, layer: int, ep_rank: Optional[int] = None) -> List[int]:
        """Logical ids of the experts that rollout expert-parallel rank ``ep_rank`` (default: this rank's)
        hosts for ``layer``, in slot order."""
        ei = self.infer_state.rank_in("ep") if ep_rank is None else ep_rank
        if self.expert_map is not None:
            entry = self.expert_map["layer_list"][self._moe_index(layer)]
            return list(entry["device_list"][ei]["device_expert"])
        n_loc = self.cfg.num_experts // self.infer_ep
        return list(range(ei * n_loc, (ei + 1) * n_loc))

    def log2phy(self, layer: int) -> Optional[torch.Tensor]:
        """``[E, max_replicas]`` physical slot ids of every logical expert (-1 padded), or ``None`` when
        slot ``i`` simply holds expert ``i``."""
        if self.expert_map is None:
            return None
        where: List[List[int]] = [[] for _ in range(self.cfg.num_experts)]
        slot = 0
        for ei in range(self.infer_ep):
            for e in self.hosted_experts(layer, ei):
                where[e].append(slot)
                slot += 1
        if any(not w for w in where):
            raise ValueError(f"the expert map hosts no copy of some expert of layer {layer}")
        width = max(len(w) for w in where)
        return torch.tensor([w + [-1] * (width - len(w)) for w in where], dtype=torch.int64)

    def _expert_placement(self) -> Optional[ExpertPlacement]:
        if not self.rehome:
            return None
        layout, me = self.train_state.layout, self.train_state.rank
        mine = layout.expert_coords(me)

        def src_rank(ep_index: int, stage: int) -> int:
            # the training rank of my own expert-data-parallel replica that owns this expert shard
            stage_rank = mine["etp"] + layout.expert_tp * (ep_index + layout.ep_total * mine["edp"])
            tp = stage_rank % layout.tp
            cp = (stage_rank // layout.tp) % layout.cp
            dp = stage_rank // (layout.tp * layout.cp)
            return layout.rank_of(tp=tp, cp=cp, dp=dp, pp=stage)

        return ExpertPlacement(self.cfg.num_experts // layout.ep_total, self.hosted_experts, src_rank)

    # ------------------------------------------------------------------------------------------
    def _main_buffer(self):
        return self.ddp.buffers[0]

    def _source_buffers(self) -> list:
        """The flat buffers that hold rollout-relevant parameters, in ``Slot.buf`` order: the trainable
        bf16 buffers (dense, then experts) and the frozen one (base weights under LoRA)."""
        dt = self._main_buffer().param_dtype
        out = [b for b in self.ddp.buffers if b.param_dtype == dt]
        frozen = getattr(self.ddp, "frozen_buffer", None)
        if frozen is not None:
            out.append(frozen)
        # parameters kept in fp32 inside a 16-bit model (routers): their buffer comes last
        out += [b for b in self.ddp.buffers if b.param_dtype != dt]
        return out

    def _home(self, buf):
        """Peer-mapped home of a flat buffer (the job-wide arena or the buffer's own segment), or
        ``None`` when it is a plain allocation."""
        return getattr(buf, "param_arena", None) if self.arena is not None else None

    def _use_arena(self) -> bool:
        return all(self._home(b) is not None for b in self._source_buffers())

    def _build(self) -> None:
        ps = self.train_state
        bufs = self._source_buffers()
        mine: Dict[str, Slot] = {}
        for bi, b in enumerate(bufs):
            for sl in b.slots:
                mine[sl.name] = Slot(sl.start, tuple(sl.shape), bi,
                                     0 if b.param_dtype == bufs[0].param_dtype else b.param_data.element_size())
        use_arena = self._use_arena()
        bases = [self._home(b).offset_of(b.param_data) if use_arena else 0 for b in bufs]
        stage = ps.rank_in("pp")
        # expert sources sit on other data-parallel ranks: their buffer offsets are needed too
        group_name = "all" if self.rehome else "mp"
        # the slot tables are the same on all tensor- and data-parallel ranks of a stage: one sender each
        sender = ps.rank_in("tp") == 0 and (not self.rehome or ps.rank_in("dp_cp") == 0)
        info = (ps.rank, stage, bases, mine if sender else None)
        if dist.is_initialized() and ps.size(group_name) > 1:
            box: List = [None] * ps.size(group_name)
            dist.all_gather_object(box, info, group=ps.group(group_name))
        else:
            box = [info]
        tables: List[Optional[Dict[str, Slot]]] = [None] * ps.size("pp")
        all_bases: Dict[int, List[int]] = {}
        for r, st, b, table in box:
            all_bases[r] = b
            if table is not None:
                tables[st] = table
        src_base = (lambda r, buf=0: all_bases[r][buf]) if use_arena else (lambda r, buf=0: 0)
        esz = bufs[0].param_data.element_size()
        self._plan = build_plan(self.cfg, ps.layout, self.infer_tp, ps.rank, tables, self._layers, src_base, esz,
                                experts=self._expert_placement())
        if use_arena:
            from ..parallel.symm import plan_to_device

            # one launch per peer-mapped home: buffers inside the job-wide arena share one, a buffer
            # with a segment of its own is read through that segment's peer pointers
            groups: Dict[int, List[Desc]] = {}
            for i, d in enumerate(self._plan.desc):
                groups.setdefault(self._plan.buf_of(i), []).append(d)
            merged: Dict[int, Tuple[int, List[Desc]]] = {}
            for bi, descs in sorted(groups.items()):
                key = id(self._home(bufs[bi]))
                merged.setdefault(key, (bi, []))[1].extend(descs)
            self._plan_dev = [(bi, plan_to_device(descs, self.device)) for bi, descs in merged.values()]

    def _moe_builder(self, core):
        if not self.rehome:
            def build(li, t):
                return core.decoder.layers[li].mlp.rollout_view()
            return build

        from ..rollout.moe import MoEWeights

        cfg = self.cfg
        h, f = cfg.hidden_size, cfg.moe_ffn_hidden_size
        ep_group = self.infer_state.group("ep") if self.infer_ep > 1 else None

        def build(li, t):
            p = f"decoder.layers.{li}.mlp."
            n_loc = len(self.hosted_experts(li))
            numbers = list(core.layer_numbers)
            layer = core.decoder.layers[numbers.index(li)].mlp if li in numbers else None
            shared = None
            if t(p + "shared_experts.linear_fc1.weight") is not None:
                shared = (t(p + "shared_experts.linear_fc1.weight"), t(p + "shared_experts.linear_fc2.weight"))
            bias = getattr(getattr(layer, "router", None), "expert_bias", None) if layer is not None else None
            table = self.log2phy(li)
            return MoEWeights(cfg, t(p + "router.weight"), t(p + "experts.weight1").view(h, n_loc, 2 * f),
                              t(p + "experts.weight2").view(n_loc, f, h), ep_group, self.infer_ep,
                              self.infer_state.rank_in("ep") if self.infer_ep > 1 else 0, shared=shared,
                              log2phy=table.to(self.device) if table is not None else None, expert_bias=bias,
                              collect_counts=bool(getattr(layer, "collect_rollout_counts", False)))
        return build

    @torch.no_grad()
    def reshard(self, core) -> RolloutWeights:
        if self._plan is None:
            self._build()
        plan = self._plan
        bufs = self._source_buffers()
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
            self._home(bufs[0]).align()
            if timed:
                self._events[0].record()
            for bi, dev_plan in self._plan_dev:
                self._home(bufs[bi]).copy_plan(dev_plan[0], dev_plan[1], self.buffer, sync=True)
        else:
            self._gathered_copy(plan, bufs)
        if timed:
            self._events[1].record()
        self.last_bytes = sum(d[3] * d[4] for d in plan.desc)
        return weights_from_buffer(self.infer_cfg, self.infer_tp, self.infer_state.rank_in("tp"), plan, self.buffer,
                                   bufs[0].param_dtype, self._moe_builder(core) if self.cfg.is_moe else None)

    def _gathered_copy(self, plan: ReshardPlan, bufs) -> None:
        """Library fallback: all-gather the parameter buffers of the ranks that hold sources (the
        model-parallel group; every rank of the job when experts move), then run the plan locally."""
        ps = self.train_state
        group_name = "all" if self.rehome else "mp"
        local = [b.param_data.view(torch.uint8) for b in bufs]
        if dist.is_initialized() and ps.size(group_name) > 1:
            sources = {}
            for bi, loc in enumerate(local):
                sizes = [None] * ps.size(group_name)
                dist.all_gather_object(sizes, int(loc.numel()), group=ps.group(group_name))
                cap = max(sizes)
                padded = torch.zeros(cap, dtype=torch.uint8, device=loc.device)
                padded[:loc.numel()] = loc
                got = [torch.empty_like(padded) for _ in sizes]
                dist.all_gather(got, padded, group=ps.group(group_name))
                for r, g in zip(ps.ranks(group_name), got):
                    sources[(r, bi)] = g
        else:
            sources = {(ps.rank, bi): loc for bi, loc in enumerate(local)}
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
