"""The rollout engine: request API, step loop and the training-framework facing wrapper.

``LLMEngine`` offers the request-level API the workers use for synchronous generation,
asynchronous streaming, partial rollout (abort + resume) and the multi-turn tool loop:
``add_request / step / abort_request / has_unfinished_requests`` (reference contract:
``mindspeed_rl/models/rollout/vllm_engine.py:506-555``,
``workers/actor_hybrid_worker.py:685-733``).

``RolloutEngine`` implements the inference-engine interface of the framework
(``init_cache_engine / free_cache_engine / sync_model_weights / offload_model_weights /
generate_sequences / async_generate_sequences``; reference:
``mindspeed_rl/models/base/base_inference_engine.py:6-125``).
"""
from __future__ import annotations

import collections
import os
import time
import uuid
import zlib
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterator, List, Optional, Sequence as Seq_, Tuple

import numpy as np
import torch

from .. import ops
from ..models.transformer_config import TransformerConfig
from ..obs.io_counter import count_d2h, to_device, to_host
from ..parallel.tp_comm import NO_TP, TPComm
from .base_engine import BaseInferEngine
from .block_manager import BlockManager
from .model_runner import KVCache, ModelRunner, RolloutWeights
from .scheduler import (PrefillItem, RequestGroup, SamplingParams, Scheduler, SchedulerOutput, SeqStatus,
                        Sequence)


@dataclass
class CompletionOutput:
    index: int
    token_ids: List[int]
    logprobs: List[float]
    finish_reason: str


@dataclass
class RequestOutput:
    request_id: str
    prompt_token_ids: List[int]
    outputs: List[CompletionOutput]
    finished: bool = True


def length_hazard(step: int, lo: int, hi: int) -> float:
    """P(stop at response length ``step``) so that lengths are uniform on ``[lo, hi]``."""
    if step < lo:
        return 0.0
    if step >= hi:
        return 1.0
    return 1.0 / (hi - step + 1)


class LLMEngine(BaseInferEngine):
    def __init__(self, cfg: TransformerConfig, device, *, max_num_seqs: int = 256,
                 max_num_batched_tokens: int = 8192, max_model_len: int = 4096, block_size: int = 16,
                 enable_prefix_caching: bool = False, enforce_eager: bool = True,
                 graph_batch_sizes: Seq_[int] = (), eos_token_id: int = -1, pad_token_id: int = 0,
                 comm: Optional[TPComm] = None, seed: int = 0, lockstep_group=None):
        """``lockstep_group``: process group whose members must run the same number of model
        forwards (the expert-parallel group of an MoE model: every forward contains all-to-all
        exchanges with the other members).  Such engines step together: a member without work
        joins the others' exchanges with zero tokens until all of them are done."""
        BaseInferEngine.__init__(self, max_num_seqs=max_num_seqs, max_model_len=max_model_len,
                                 infer_tensor_parallel_size=(comm.world_size if comm is not None else 1))
        self.cfg = cfg
        self.lockstep_group = lockstep_group
        self.device = torch.device(device)
        self.comm = comm or NO_TP
        self.max_num_seqs, self.max_num_batched_tokens = max_num_seqs, max_num_batched_tokens
        self.max_model_len, self.block_size = max_model_len, block_size
        self.enable_prefix_caching = enable_prefix_caching
        self.eos_token_id, self.pad_token_id = eos_token_id, pad_token_id
        self.seed = seed
        self.runner = ModelRunner(cfg, device, self.comm, max_model_len, enforce_eager,
                                  tuple(b for b in graph_batch_sizes if b <= max_num_seqs))
        self.bm: Optional[BlockManager] = None
        self.scheduler: Optional[Scheduler] = None
        self._step_counter = 0
        self.host_time = collections.defaultdict(float)   # wall-clock seconds per host-side section
        nkv_local = max(cfg.num_query_groups // self.comm.world_size, 1)
        nh_local = cfg.num_attention_heads // self.comm.world_size
        # shared prompts are rounded down to the tensor-core prefix kernel's key tile (0: the mma.sync kernel takes any length)
        self._prefix_tile = ops.decode_prefix_tile(nh_local, nkv_local, cfg.head_dim, block_size) \
            if torch.device(device).type == "cuda" else 0
        self.runner.prefix_tile = self._prefix_tile
        self._group_max = ops.decode_group_max(nh_local, nkv_local, self._prefix_tile)
        self.shared_prefix_decode = os.environ.get("MSRL_SHARED_PREFIX_DECODE", "1") == "1"
        self.lookahead_decode = os.environ.get("MSRL_LOOKAHEAD_DECODE", "1") == "1" and lockstep_group is None
        self.stats = dict(prefill_tokens=0, decode_tokens=0, steps=0, preemptions=0, lookahead_steps=0)

    # ---- cache lifecycle -----------------------------------------------------------------------
    def kv_bytes_per_block(self) -> int:
        c = self.cfg
        nkv = c.num_query_groups // self.comm.world_size
        return KVCache.bytes_per_block(c.num_layers, self.block_size, nkv, c.head_dim, c.params_dtype)

    def init_cache(self, num_blocks: int) -> None:
        c = self.cfg
        nkv = c.num_query_groups // self.comm.world_size
        cache = KVCache(c.num_layers, num_blocks, self.block_size, nkv, c.head_dim, c.params_dtype,
                        self.device)
        self.runner.bind_cache(cache)
        self.bm = BlockManager(num_blocks, self.block_size, self.enable_prefix_caching)
        self.scheduler = Scheduler(self.bm, self.max_num_seqs, self.max_num_batched_tokens,
                                   self.max_model_len)

    def free_cache(self) -> None:
        if os.environ.get("MSRL_ENGINE_PROFILE", "0") == "1" and self.host_time:
            print("[engine] steps=%d (launched ahead: %d) host seconds: %s" % (
                self.stats["steps"], self.stats.get("lookahead_steps", 0),
                {k: round(v, 3) for k, v in sorted(self.host_time.items())}), flush=True)
            self.host_time.clear()
        self.runner.bind_cache(None)
        self.bm = None
        self.scheduler = None

    # ---- the worker-facing contract (BaseInferEngine) ---------------------------------------------
    def init_cache_engine(self, num_blocks: Optional[int] = None) -> None:
        self.init_cache(num_blocks if num_blocks is not None else getattr(self, "default_num_blocks", 0))

    def free_cache_engine(self) -> None:
        self.free_cache()

    def offload_model_weights(self) -> None:
        self.runner.bind_weights(None)

    def sync_model_weights(self, params, load_format: str = "megatron") -> None:
        """``params``: a ``RolloutWeights`` view of the training tensors (aliased or resharded)."""
        self.runner.bind_weights(params)

    def generate_sequences(self, idx_list, sampling_params=None, **kwargs):
        return self.generate(idx_list, sampling_params or SamplingParams(**kwargs))

    # ---- request API ---------------------------------------------------------------------------
    def add_request(self, request_id: Optional[str], prompt_token_ids: Seq_[int],
                    params: SamplingParams, mm: Optional[dict] = None) -> str:
        """``mm`` (vision-language prompt): ``dict(vit_embeds [n, H], position_ids [P, 3], image_token_id)``;
        the placeholder tokens' embeddings are replaced by the rows of ``vit_embeds`` in the prefill."""
        # generated ids must be the same on every rank of a rollout TP group (they seed the
        # per-request sampling stream, and the ranks must draw the same tokens): a counter, not a uuid
        self._request_counter = getattr(self, "_request_counter", 0) + 1
        rid = request_id or f"req-{self._request_counter:010d}"
        if rid in self.scheduler.groups:
            raise ValueError(f"request id {rid} is already in flight")
        lead = Sequence(rid, list(int(t) for t in prompt_token_ids), params, sample_index=0)
        if mm is not None and mm.get("vit_embeds") is not None:
            if self.enable_prefix_caching:
                raise ValueError("prefix caching keys blocks by token ids only and cannot tell two images apart; "
                                 "turn enable_prefix_caching off for vision-language rollouts")
            self.image_token_id = int(mm.get("image_token_id", 151655))
            lead.mm_embeds = mm["vit_embeds"]
            pos3 = mm.get("position_ids")
            if pos3 is not None:
                lead.mm_positions = pos3[:len(lead.prompt_ids)]
                lead.pos_delta = int(lead.mm_positions.max()) + 1 - len(lead.prompt_ids) if len(lead.prompt_ids) else 0
        self.scheduler.add_group(RequestGroup(rid, params, [lead]))
        return rid

    def abort_request(self, request_id: str) -> Optional[RequestOutput]:
        group = self.scheduler.groups.get(request_id)
        if group is None:
            return None
        self.scheduler.abort(request_id)
        self.scheduler.groups.pop(request_id, None)
        return self._to_output(group)

    def has_unfinished_requests(self) -> bool:
        return self.scheduler is not None and self.scheduler.has_unfinished()

    def any_unfinished_requests(self) -> bool:
        """Collective over the lock-step group (every member must call it once per step): true
        while any member still has requests."""
        mine = self.has_unfinished_requests()
        if self.lockstep_group is None:
            return mine
        flag = torch.tensor([1 if mine else 0], dtype=torch.int32, device=self.device)
        torch.distributed.all_reduce(flag, op=torch.distributed.ReduceOp.MAX, group=self.lockstep_group)
        return bool(flag.item())

    def get_num_unfinished_requests(self) -> int:
        return len(self.scheduler.groups)

    # ---- one engine step -----------------------------------------------------------------------
    def step(self) -> List[RequestOutput]:
        t0 = time.perf_counter()
        sched = self.scheduler.schedule()
        t1 = time.perf_counter()
        self.stats["steps"] += 1
        self.stats["preemptions"] += len(sched.preempted)
        if sched.prefill:
            self._run_prefill(sched.prefill)
            self.host_time["prefill_step"] += time.perf_counter() - t1
        elif sched.decode:
            self._run_decode(sched.decode)
            self.host_time["decode_step"] += time.perf_counter() - t1
        elif self.lockstep_group is not None:
            self.runner.idle_forward()            # keep the other members' exchanges paired
            self.stats["idle_steps"] = self.stats.get("idle_steps", 0) + 1
        self._step_counter += 1
        t2 = time.perf_counter()
        out = [self._to_output(g) for g in self.scheduler.pop_finished_groups()]
        self.host_time["schedule"] += t1 - t0
        self.host_time["collect"] += time.perf_counter() - t2
        return out

    # ---- internals -----------------------------------------------------------------------------
    def _ship(self, ints: List[List[int]], floats: Optional[List[List[float]]] = None):
        """Send several equally long integer (and float) rows in ONE pinned copy each."""
        dev = self.device
        it = to_device(np.asarray(ints, dtype=np.int64), torch.int64, dev)
        ft = to_device(np.asarray(floats, dtype=np.float32), torch.float32, dev) if floats else None
        return it, ft

    def _sampling_rows(self, seqs: List[Sequence], pend: int = 0):
        """Host-side sampling parameters: (row_keys, float rows, flags).  ``pend``: tokens sampled
        but not yet appended on the host."""
        keys, temp = [], []
        need_filter = need_eos = False
        for s in seqs:
            p = s.params
            base = p.seed if p.seed is not None else (zlib.crc32(s.request_id.encode()) & 0x7FFFFFFF)
            keys.append(((base * 1000003 + s.sample_index) * 1000003 + len(s.output_ids) + pend) & (2 ** 62 - 1))
            temp.append(p.temperature)
            need_filter |= p.top_k > 0 or p.top_p < 1.0 or p.min_p > 0.0
            need_eos |= p.eos_hazard is not None
        floats = [temp]
        if need_filter:
            floats += [[float(max(s.params.top_k, 0)) for s in seqs], [s.params.top_p for s in seqs],
                       [s.params.min_p for s in seqs]]
        if need_eos:
            floats.append([length_hazard(len(s.output_ids) + 1 + pend, *s.params.eos_hazard)
                           if s.params.eos_hazard is not None else -1.0 for s in seqs])
        return keys, floats, need_filter, need_eos

    def _sample(self, logits: torch.Tensor, seqs: List[Sequence], keys: torch.Tensor,
                ft: torch.Tensor, need_filter: bool, need_eos: bool) -> Tuple[List[int], List[float]]:
        tokens, logprobs = self._sample_device(logits, keys, ft, need_filter, need_eos)
        # one device->host read per step: tokens and their log-probs together
        both = to_host(torch.stack([tokens.double(), logprobs.double()]))
        return both[0].long().tolist(), both[1].tolist()

    def _sample_device(self, logits: torch.Tensor, keys: torch.Tensor, ft: torch.Tensor, need_filter: bool,
                       need_eos: bool) -> Tuple[torch.Tensor, torch.Tensor]:
        temp = ft[0]
        top_k = top_p = min_p = eos_prob = None
        row = 1
        if need_filter:
            top_k, top_p, min_p = ft[1].to(torch.int32), ft[2], ft[3]
            row = 4
        if need_eos:
            eos_prob = ft[row]
        if self.comm.world_size > 1:  # vocabulary-sharded head: gather the logits of the few rows
            parts = [torch.empty_like(logits) for _ in range(self.comm.world_size)]
            torch.distributed.all_gather(parts, logits.contiguous(), group=self.comm.group)
            logits = torch.cat(parts, dim=-1)
        return ops.sample(logits, temp, top_k, top_p, min_p, keys, self.seed, eos_prob, self.eos_token_id)

    def _append_token(self, seq: Sequence, token: int, logprob: float) -> None:
        seq.output_ids.append(int(token))
        seq.output_logprobs.append(float(logprob))
        p = seq.params
        if not p.ignore_eos and (token == self.eos_token_id or token in p.stop_token_ids):
            self.scheduler.finish(seq, SeqStatus.FINISHED_STOPPED)
        elif len(seq.output_ids) >= p.max_tokens or seq.total_len >= self.max_model_len:
            self.scheduler.finish(seq, SeqStatus.FINISHED_LENGTH)

    def _run_prefill(self, items: List[PrefillItem]) -> None:
        dev = self.device
        ids, pos, slots, cu, last_rows, finishing = [], [], [], [0], [], []
        need_prefix = any(it.start > 0 for it in items)
        tok_seq, tok_pos, cu_k = [], [], [0]
        for row, it in enumerate(items):
            s = it.seq
            all_ids = s.all_ids
            ids.extend(all_ids[it.start:it.start + it.length])
            pos.extend(range(it.start, it.start + it.length))
            slots.append(self.bm.slots(s.seq_id, it.start, it.length))
            cu.append(cu[-1] + it.length)
            if it.completes_prompt:
                last_rows.append(cu[-1] - 1)
                finishing.append(s)
            if need_prefix:
                end = it.start + it.length
                tok_seq.extend([row] * end)
                tok_pos.extend(range(end))
                cu_k.append(cu_k[-1] + end)
        tok, _ = self._ship([ids, pos, np.concatenate(slots).tolist()])
        t_ids, t_pos, t_slots = tok[0], tok[1].to(torch.int32), tok[2]
        t_cu = to_device(cu, torch.int32, dev)
        t_last = to_device(last_rows, torch.int64, dev)
        prefix = None
        if need_prefix:
            max_blocks = max(len(self.bm.block_table(it.seq.seq_id)) for it in items)
            bt = self.bm.block_tables([it.seq.seq_id for it in items], max_blocks)
            pt, _ = self._ship([tok_seq, tok_pos])
            prefix = dict(block_tables=to_device(bt, torch.int32, dev), token_seq=pt[0].to(torch.int32),
                          token_pos=pt[1].to(torch.int32), cu_k=to_device(cu_k, torch.int32, dev))
        logits = self.runner.prefill(t_ids, t_pos, t_slots, t_cu, max(it.length for it in items), t_last,
                                     prefix, self._prefill_mm(items, ids, pos))
        self.stats["prefill_tokens"] += len(ids)
        for it in items:
            it.seq.num_computed = it.start + it.length
            self.bm.commit(it.seq.seq_id, it.seq.all_ids, it.seq.num_computed)
        if not finishing:
            return
        # fork n-sample groups, then sample one token per resulting sequence
        rows, seqs = [], []
        for r, lead in enumerate(finishing):
            rows.append(r)
            seqs.append(lead)
            group = self.scheduler.groups.get(lead.request_id)
            if group is not None and not group.forked:
                for child, (src, dst) in self.scheduler.fork_group(lead):
                    if src >= 0:
                        self.runner.cache.copy_block(src, dst)
                    rows.append(r)
                    seqs.append(child)
        keys, floats, need_filter, need_eos = self._sampling_rows(seqs)
        it_, ft = self._ship([keys, rows], floats)
        sel = logits if rows == list(range(logits.shape[0])) else logits[it_[1]]
        tokens, lps = self._sample(sel, seqs, it_[0], ft, need_filter, need_eos)
        for s, tok_, lp in zip(seqs, tokens, lps):
            self._append_token(s, tok_, lp)

    def _prefill_mm(self, items, ids: List[int], pos: List[int]) -> Optional[dict]:
        """Vision-language part of a prefill batch (``None`` for text-only batches): packed positions of the
        image placeholder tokens with their embedding rows, and the per-token rotary table."""
        if not any(it.seq.mm_embeds is not None for it in items):
            return None
        from ..datasets.mm_utils import extend_positions, mrope_table

        index, rows, pos3, base = [], [], [], 0
        for it in items:
            s = it.seq
            chunk = ids[base:base + it.length]
            if s.mm_embeds is not None:
                tok = self.image_token_id
                before = sum(1 for t in s.all_ids[:it.start] if t == tok)       # placeholders of earlier chunks
                where = [j for j, t in enumerate(chunk) if t == tok]
                if where:
                    index.extend(base + j for j in where)
                    rows.append(s.mm_embeds[before:before + len(where)])
            if s.mm_positions is not None:
                full = extend_positions(s.mm_positions, max(it.start + it.length - s.mm_positions.shape[0], 0))
                pos3.append(full[it.start:it.start + it.length])
            else:
                pos3.append(torch.tensor(pos[base:base + it.length]).unsqueeze(-1).expand(-1, 3))
            base += it.length
        dev = self.device
        table = mrope_table(torch.cat(pos3), self.runner.rope_table())
        out = dict(rope_table=table.to(dev))
        if index:
            out["image_index"] = to_device(index, torch.int64, dev)
            out["image_embeds"] = torch.cat(rows).to(dev)
        return out

    def _launch_decode(self, seqs: List[Sequence], prev: Optional[dict] = None) -> dict:
        """Launch one decode step and its sampling; nothing is read back.

        ``prev``: the step still in flight whose sampled tokens (on the device) are this step's
        input ids; host-side lengths then count that pending token."""
        dev = self.device
        b = len(seqs)
        t0 = time.perf_counter()
        pend = 0 if prev is None else 1
        lens = [s.total_len + pend for s in seqs]
        slots = [int(self.bm.slots(s.seq_id, n - 1, 1)[0]) for s, n in zip(seqs, lens)]
        keys, floats, need_filter, need_eos = self._sampling_rows(seqs, pend)
        if prev is None:
            last = [s.output_ids[-1] if s.output_ids else s.prompt_ids[-1] for s in seqs]
        else:
            row_of = {id(s): i for i, s in enumerate(prev["seqs"])}
            last = [row_of[id(s)] for s in seqs]          # rows of the pending step's token tensor
        rows = [last, [n - 1 + s.pos_delta for s, n in zip(seqs, lens)], slots, lens, keys]
        grouped = False
        if self.shared_prefix_decode and dev.type == "cuda":
            # samples of one prompt share the prompt's K/V: read it once per group
            ks, grows, gpre, grouped = ops.build_decode_groups(
                [s.request_id for s in seqs], [len(s.prompt_ids) for s in seqs], self._group_max,
                multiple=max(1, self._prefix_tile))
            if grouped:
                rows += [ks, gpre] + [list(col) for col in zip(*grows)]
        t1 = time.perf_counter()
        it_, ft = self._ship(rows, floats)
        max_ctx = max(lens)
        max_blocks = (max_ctx + self.block_size - 1) // self.block_size
        bt = to_device(self.bm.block_tables([s.seq_id for s in seqs], max_blocks), torch.int32, dev)
        groups = None
        if grouped:
            groups = (it_[5].to(torch.int32), it_[7:15].t().contiguous().to(torch.int32), it_[6].to(torch.int32),
                      sum(1 for grp in grows if grp[0] >= 0))
        ids = it_[0]
        if prev is not None:
            ids = prev["tokens"] if last == list(range(len(prev["seqs"]))) else prev["tokens"][it_[0]]
        t2 = time.perf_counter()
        logits = self.runner.decode(ids, it_[1].to(torch.int32), it_[2], bt, it_[3].to(torch.int32), max_ctx, groups)
        self.stats["decode_tokens"] += b
        tokens, logprobs = self._sample_device(logits, it_[4], ft, need_filter, need_eos)
        tokens = tokens.long()
        both = torch.stack([tokens.double(), logprobs.double()])
        event = None
        if both.is_cuda:
            host = torch.empty(both.shape, dtype=both.dtype, pin_memory=True)
            host.copy_(both, non_blocking=True)
            event = torch.cuda.Event()
            event.record()
            count_d2h(both.numel() * both.element_size())
        else:
            host = both
        ht = self.host_time
        ht["decode_prep"] += t1 - t0
        ht["decode_h2d"] += t2 - t1
        ht["decode_launch"] += time.perf_counter() - t2
        return dict(seqs=seqs, lens=lens, tokens=tokens, host=host, event=event)

    def _finish_decode(self, h: dict) -> None:
        """Read a launched step's tokens and append them; sequences that finished while the step
        was in flight (end of sequence found in the step before) drop their extra token."""
        t0 = time.perf_counter()
        if h["event"] is not None:
            h["event"].synchronize()
        tokens, lps = h["host"][0].long().tolist(), h["host"][1].tolist()
        t1 = time.perf_counter()
        for s, n, tok, lp in zip(h["seqs"], h["lens"], tokens, lps):
            if s.finished:
                continue
            s.num_computed = n
            self._append_token(s, tok, lp)
        self.host_time["decode_sample_sync"] += t1 - t0      # includes waiting for the GPU to finish the step
        self.host_time["decode_append"] += time.perf_counter() - t1

    def _may_look_ahead(self, seqs: List[Sequence]) -> List[Sequence]:
        """Sequences whose next decode step can be launched before this step's tokens are known:
        nothing waits for a prefill, the batch is the whole running set, every sequence outlives
        the pending token by length, and the block pool covers their next slots."""
        sch = self.scheduler
        if not self.lookahead_decode or sch.waiting or len(seqs) != len(sch.running):
            return []
        cont = [s for s in seqs
                if len(s.output_ids) + 1 < s.params.max_tokens and s.total_len + 1 < self.max_model_len]
        if len(cont) != len(seqs):
            return []          # a sequence ends by length: let the scheduler regroup first
        need = sum(self.bm.blocks_needed(s.seq_id, s.total_len + 1) for s in cont)
        if need > self.bm.num_free_blocks:
            return []
        return cont

    def _run_decode(self, seqs: List[Sequence]) -> None:
        """One scheduled decode step, then further steps launched one ahead of the host: step i+1
        takes its input ids from step i's token tensor on the device, so the host prepares and
        launches it while step i still runs and reads step i's tokens afterwards.  A sequence that
        turns out to have ended in step i has one surplus token computed; it is dropped."""
        h = self._launch_decode(seqs)
        while True:
            cont = self._may_look_ahead(h["seqs"])
            if not cont:
                break
            for s in cont:
                self.bm.append(s.seq_id, 1)       # slot of the pending token
            nxt = self._launch_decode(cont, h)
            self._finish_decode(h)
            self.stats["steps"] += 1
            self.stats["lookahead_steps"] += 1
            self._step_counter += 1
            h = nxt
            if any(s.finished for s in cont):
                break                              # regroup without the finished sequences
        self._finish_decode(h)

    def _to_output(self, group: RequestGroup) -> RequestOutput:
        reasons = {SeqStatus.FINISHED_STOPPED: "stop", SeqStatus.FINISHED_LENGTH: "length",
                   SeqStatus.FINISHED_ABORTED: "abort"}
        outs = [CompletionOutput(s.sample_index, list(s.output_ids), list(s.output_logprobs),
                                 reasons.get(s.status, "abort"))
                for s in sorted(group.seqs, key=lambda x: x.sample_index)]
        return RequestOutput(group.request_id, list(group.seqs[0].prompt_ids), outs, True)

    # ---- convenience -----------------------------------------------------------------------------
    def generate(self, prompts: Seq_[Seq_[int]], params: SamplingParams,
                 request_ids: Optional[Seq_[str]] = None, mm: Optional[Seq_[Optional[dict]]] = None
                 ) -> List[RequestOutput]:
        """Blocking generation; results come back in the order of ``prompts``.  ``params`` may be
        one ``SamplingParams`` or a list with one entry per prompt."""
        per_prompt = isinstance(params, (list, tuple))
        rids = [self.add_request(None if request_ids is None else request_ids[i], p,
                                 params[i] if per_prompt else params, None if mm is None else mm[i])
                for i, p in enumerate(prompts)]
        done: Dict[str, RequestOutput] = {}
        while self.any_unfinished_requests():
            for out in self.step():
                done[out.request_id] = out
        for g in self.scheduler.pop_finished_groups():
            done[g.request_id] = self._to_output(g)
        return [done[r] for r in rids]
