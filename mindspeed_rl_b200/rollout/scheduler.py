"""Requests, sequences and the continuous-batching scheduler of the rollout engine.

Scheduling policy: prefill first (prompts are admitted FIFO under the token budget
``max_num_batched_tokens`` and the sequence cap ``max_num_seqs``; long prompts are split
into chunks across steps), otherwise one decode step over every running sequence.  When the
KV cache runs out of blocks during decode, the most recently admitted sequence is preempted:
its blocks are released and it re-enters the waiting queue with ``prompt + generated so far``
as its new prompt (recompute policy).  A request that asks for ``n`` samples prefills its
prompt once; the ``n`` sequences are forked from it and share the prompt's KV blocks.
"""
from __future__ import annotations

import enum
import itertools
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Tuple

from .block_manager import BlockManager, OutOfBlocks


@dataclass
class SamplingParams:
    n: int = 1
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    min_p: float = 0.0
    max_tokens: int = 128
    seed: Optional[int] = None
    logprobs: Optional[int] = 1
    detokenize: bool = False
    stop_token_ids: Tuple[int, ...] = ()
    ignore_eos: bool = False
    # benchmark length control: P(eos at step t) = hazard(t); see engine.length_hazard
    eos_hazard: Optional[Tuple[int, int]] = None   # (min_len, max_len): uniform length on [min, max]

    @classmethod
    def from_config(cls, sampling_config: dict, **overrides) -> "SamplingParams":
        kw = {k: v for k, v in dict(sampling_config).items() if k in cls.__dataclass_fields__}
        kw.update(overrides)
        if kw.get("top_k") in (None, 0):
            kw["top_k"] = -1
        return cls(**kw)


class SeqStatus(enum.Enum):
    WAITING = 0
    RUNNING = 1
    FINISHED_STOPPED = 2
    FINISHED_LENGTH = 3
    FINISHED_ABORTED = 4

    @property
    def finished(self) -> bool:
        return self.value >= 2


_seq_counter = itertools.count()


@dataclass
class Sequence:
    request_id: str
    prompt_ids: List[int]
    params: SamplingParams
    sample_index: int = 0
    seq_id: int = field(default_factory=lambda: next(_seq_counter))
    output_ids: List[int] = field(default_factory=list)
    output_logprobs: List[float] = field(default_factory=list)
    status: SeqStatus = SeqStatus.WAITING
    num_computed: int = 0          # tokens whose KV is in the cache
    num_preemptions: int = 0
    prefill_target: int = 0        # tokens to prefill since the last admission
    arrival: int = 0
    # vision-language prompts: rows of the vision tower for the image placeholder tokens (in order),
    # three-axis positions of the prompt, and what decoding adds to its one-axis position counter
    mm_embeds: Optional[object] = None
    mm_positions: Optional[object] = None
    pos_delta: int = 0

    @property
    def all_ids(self) -> List[int]:
        return self.prompt_ids + self.output_ids

    @property
    def total_len(self) -> int:
        return len(self.prompt_ids) + len(self.output_ids)

    @property
    def finished(self) -> bool:
        return self.status.finished


@dataclass
class RequestGroup:
    request_id: str
    params: SamplingParams
    seqs: List[Sequence]
    forked: bool = False

    @property
    def finished(self) -> bool:
        return self.forked and all(s.finished for s in self.seqs)


@dataclass
class PrefillItem:
    seq: Sequence
    start: int
    length: int

    @property
    def completes_prompt(self) -> bool:
        return self.start + self.length >= self.seq.prefill_target


@dataclass
class SchedulerOutput:
    prefill: List[PrefillItem] = field(default_factory=list)
    decode: List[Sequence] = field(default_factory=list)
    preempted: List[Sequence] = field(default_factory=list)

    @property
    def empty(self) -> bool:
        return not self.prefill and not self.decode


class Scheduler:
    def __init__(self, block_manager: BlockManager, max_num_seqs: int, max_num_batched_tokens: int,
                 max_model_len: int):
        self.bm = block_manager
        self.max_num_seqs = max_num_seqs
        self.max_num_batched_tokens = max_num_batched_tokens
        self.max_model_len = max_model_len
        self.waiting: Deque[Sequence] = deque()
        self.running: List[Sequence] = []
        self.groups: Dict[str, RequestGroup] = {}
        self._clock = itertools.count()
        self._allocated: set = set()

    # ------------------------------------------------------------------------------------------
    def add_group(self, group: RequestGroup) -> None:
        self.groups[group.request_id] = group
        lead = group.seqs[0]
        lead.arrival = next(self._clock)
        self.waiting.append(lead)

    def abort(self, request_id: str) -> List[Sequence]:
        group = self.groups.get(request_id)
        if group is None:
            return []
        out = []
        for s in group.seqs:
            if not s.finished:
                s.status = SeqStatus.FINISHED_ABORTED
                self._release(s)
                out.append(s)
        self.waiting = deque(s for s in self.waiting if s.request_id != request_id)
        self.running = [s for s in self.running if s.request_id != request_id]
        group.forked = True
        return out

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    def num_unfinished(self) -> int:
        return len(self.waiting) + len(self.running)

    def _release(self, seq: Sequence) -> None:
        if seq.seq_id in self._allocated:
            self.bm.free(seq.seq_id)
            self._allocated.discard(seq.seq_id)

    def finish(self, seq: Sequence, status: SeqStatus) -> None:
        seq.status = status
        self._release(seq)
        if seq in self.running:
            self.running.remove(seq)

    def pop_finished_groups(self) -> List[RequestGroup]:
        done = [g for g in self.groups.values() if g.finished]
        for g in done:
            del self.groups[g.request_id]
        return done

    # ------------------------------------------------------------------------------------------
    def _reserve_children(self, seq: Sequence) -> int:
        """Sequences this waiting item will turn into once its prompt is done."""
        g = self.groups.get(seq.request_id)
        return g.params.n if (g is not None and not g.forked) else 1

    def schedule(self) -> SchedulerOutput:
        """Pick the work of the next engine step.

        Invariant kept with the block manager: a running sequence has slots reserved for
        ``prefill_target`` tokens while it prefills and for ``total_len - 1`` tokens between decode
        steps (the newest sampled token gets its slot when it is scheduled for decode).
        """
        out = SchedulerOutput()
        # ---- prefill -------------------------------------------------------------------------------
        budget = self.max_num_batched_tokens
        for s in self.running:  # chunked prefills in flight continue first
            if s.num_computed < s.prefill_target and budget > 0:
                n = min(budget, s.prefill_target - s.num_computed)
                out.prefill.append(PrefillItem(s, s.num_computed, n))
                budget -= n
        slots_left = self.max_num_seqs - len(self.running)
        while self.waiting and budget > 0:
            s = self.waiting[0]
            need_seqs = self._reserve_children(s)
            if need_seqs > slots_left and self.running:
                break
            if s.total_len >= self.max_model_len:
                self.waiting.popleft()
                self.finish(s, SeqStatus.FINISHED_LENGTH)
                if s.request_id in self.groups:
                    self.groups[s.request_id].forked = True
                continue
            try:
                cached = self.bm.allocate(s.seq_id, s.all_ids)
            except OutOfBlocks:
                break
            self._allocated.add(s.seq_id)
            self.waiting.popleft()
            s.status = SeqStatus.RUNNING
            s.num_computed = cached
            s.prefill_target = s.total_len
            self.running.append(s)
            slots_left -= need_seqs
            n = min(budget, s.prefill_target - s.num_computed)
            out.prefill.append(PrefillItem(s, s.num_computed, n))
            budget -= n
        if out.prefill:
            return out
        # ---- decode --------------------------------------------------------------------------------
        ready = sorted(self.running, key=lambda s: s.arrival)
        while ready:
            need = sum(self.bm.blocks_needed(s.seq_id, s.total_len) for s in ready)
            if need <= self.bm.num_free_blocks:
                for s in ready:
                    self.bm.append(s.seq_id, 1)
                break
            victim = ready.pop()  # newest
            self._preempt(victim)
            out.preempted.append(victim)
        out.decode = ready
        return out

    def _preempt(self, seq: Sequence) -> None:
        self._release(seq)
        self.running.remove(seq)
        seq.status = SeqStatus.WAITING
        seq.num_computed = 0
        seq.num_preemptions += 1
        self.waiting.appendleft(seq)

    # ------------------------------------------------------------------------------------------
    def fork_group(self, lead: Sequence) -> List[Tuple[Sequence, Tuple[int, int]]]:
        """After the lead's prompt is prefilled: create the other ``n-1`` sequences sharing its
        blocks. Returns ``[(child, (src_block, dst_block))]`` for the partial-block copies."""
        g = self.groups[lead.request_id]
        if g.forked:
            return []
        g.forked = True
        created = []
        for i in range(1, g.params.n):
            child = Sequence(lead.request_id, list(lead.prompt_ids), g.params, sample_index=i)
            child.mm_embeds, child.mm_positions, child.pos_delta = lead.mm_embeds, lead.mm_positions, lead.pos_delta
            child.arrival = next(self._clock)
            child.status = SeqStatus.RUNNING
            child.num_computed = lead.num_computed
            pair = self.bm.fork(lead.seq_id, child.seq_id)
            self._allocated.add(child.seq_id)
            g.seqs.append(child)
            self.running.append(child)
            created.append((child, pair))
        return created
