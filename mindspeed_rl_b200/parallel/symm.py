"""Symmetric memory over NVLink: one peer-mapped arena per rank and the collectives on it.

Every rank of a team (the ranks of one NVSwitch domain) allocates an arena of the same size
straight from the CUDA driver, exports it through a CUDA IPC handle and maps all peers' arenas
into its own address space.  Tensors carved out of the arena sit at the same offset on every
rank, so a kernel can address "the same tensor on rank r" as ``peer_base[r] + offset`` and move
data with plain loads and stores through NVSwitch.

The flat parameter and gradient buffers of the training model live in the arena, which lets

* the gradient reduce-scatter and parameter all-gather of the distributed optimizer
  (reference: Megatron ``DistributedOptimizer`` collectives driven from
  ``mindspeed_rl/workers/resharding/megatron_sharding_manager.py``), and
* the train -> rollout weight resharding (reference:
  ``mindspeed_rl/workers/resharding/vllm_weight_container.py:187-441``)

run as single pull kernels instead of chains of library collectives and copies.

Peer memory is only ever touched by this package's own kernels: a peer pointer never becomes
a ``torch.Tensor`` and is never handed to a library kernel.

Synchronisation is a device-side epoch barrier (flags in the arena, bounded spin).  A barrier
that runs out of time records ``100 + peer`` in the arena's status word; ``check()`` reads it.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.distributed as dist

from ..ops import _lib

_HEADER_BYTES = 4096          # flags (one u32 per rank) live at the start of every arena


class ArenaUnavailable(RuntimeError):
    """Peer-mapped memory could not be set up on at least one rank; raised on EVERY rank of the team,
    so that all of them fall back to collectives together."""


class SymmetricTimeout(RuntimeError):
    pass


class _Span:
    """Adapter that lets torch wrap a raw device range without taking ownership."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 3, "strides": None}
        self._owner = owner


def _align(n: int, a: int) -> int:
    return (n + a - 1) // a * a


class SymmetricArena:
    """``nbytes`` of peer-mapped device memory on each rank of ``group``."""

    def __init__(self, nbytes: int, group=None, device: Optional[torch.device] = None):
        if not torch.cuda.is_available():
            raise RuntimeError("symmetric memory needs CUDA devices")
        self.lib = _lib.load()
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        if self.world > int(self.lib.msrl_symm_max_ranks()):
            raise ValueError(f"a symmetric team holds at most {self.lib.msrl_symm_max_ranks()} ranks")
        self.nbytes = _align(int(nbytes) + _HEADER_BYTES, 1 << 21)
        handle = (ctypes.c_ubyte * 64)()
        base = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            rc = int(self.lib.msrl_symm_alloc(ctypes.c_longlong(self.nbytes), ctypes.byref(base), handle))
        self.base = int(base.value) if rc == 0 else 0
        self.peer_base: List[int] = [0] * self.world
        self.peer_base[self.rank] = self.base
        self._closed = False
        if self.world == 1 and rc != 0:
            raise ArenaUnavailable(f"allocation of {self.nbytes} bytes failed (CUDA error {rc})")
        if self.world > 1:
            # a failure on one rank must become the same exception on all of them (no rank may be left
            # waiting in a collective): exchange the outcome together with the handles, then the
            # outcome of mapping the peers
            handles: List[Optional[bytes]] = [None] * self.world
            dist.all_gather_object(handles, bytes(handle) if rc == 0 else None, group=group)
            failed = [r for r, h in enumerate(handles) if h is None]
            opened = 0
            if not failed:
                with torch.cuda.device(self.device):
                    for r, h in enumerate(handles):
                        if r == self.rank:
                            continue
                        p = ctypes.c_void_p()
                        buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
                        if int(self.lib.msrl_symm_open(buf, ctypes.byref(p))) != 0:
                            break
                        self.peer_base[r] = int(p.value)
                        opened += 1
            ok = [None] * self.world
            dist.all_gather_object(ok, (not failed) and opened == self.world - 1, group=group)
            if not all(ok):
                self._release()
                raise ArenaUnavailable(f"peer-mapped memory unavailable (allocation failed on ranks {failed}, "
                                       f"mapping ok per rank: {ok})")
        self._cursor = _HEADER_BYTES
        self._epochs = [0] * self.world
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._whole = torch.as_tensor(_Span(self.base, self.nbytes, self), device=self.device)
        if self.world > 1:
            dist.barrier(group=group)        # every arena is zeroed and mapped before first use

    # ---- carving ---------------------------------------------------------------------------------
    def alloc(self, shape, dtype: torch.dtype, align: int = 256) -> torch.Tensor:
        """A tensor at the same arena offset on every rank (call in the same order everywhere)."""
        shape = (shape,) if isinstance(shape, int) else tuple(shape)
        n = int(np.prod(shape)) if shape else 1
        esz = torch.empty(0, dtype=dtype).element_size()
        start = _align(self._cursor, align)
        end = start + n * esz
        if end > self.nbytes:
            raise MemoryError(f"symmetric arena exhausted: need {end} of {self.nbytes} bytes")
        self._cursor = end
        return self._whole[start:end].view(dtype).view(shape)

    def free_bytes(self) -> int:
        return self.nbytes - self._cursor

    def offset_of(self, t: torch.Tensor) -> int:
        off = t.data_ptr() - self.base
        if off < 0 or off + t.numel() * t.element_size() > self.nbytes:
            raise ValueError("tensor does not live in this arena")
        return off

    def contains(self, t: torch.Tensor) -> bool:
        off = t.data_ptr() - self.base
        return 0 <= off and off + t.numel() * t.element_size() <= self.nbytes

    def peer_ptrs(self, offset: int = 0, ranks: Optional[Sequence[int]] = None):
        """ctypes array of the members' addresses of arena offset ``offset`` (whole team by default)."""
        members = range(self.world) if ranks is None else ranks
        return (ctypes.c_void_p * len(members))(*[self.peer_base[r] + offset for r in members])

    def team_ranks(self, group) -> List[int]:
        """Positions inside this arena's team of the members of process group ``group``."""
        members = dist.get_process_group_ranks(group)
        if self.group is None:
            return list(members)
        team = dist.get_process_group_ranks(self.group)
        return [team.index(m) for m in members]

    def _members(self, ranks: Optional[Sequence[int]]) -> Tuple[List[int], int]:
        members = list(range(self.world)) if ranks is None else list(ranks)
        if self.rank not in members:
            raise ValueError("this rank is not a member of the sub-team")
        return members, members.index(self.rank)

    # ---- synchronisation ------------------------------------------------------------------------------
    def barrier(self, ranks: Optional[Sequence[int]] = None) -> None:
        """Device-side barrier on the current stream among ``ranks`` (team ranks; default all):
        kernels enqueued before it on every member are complete (and their writes visible)
        before anything enqueued after it starts.  Every pair of ranks must issue the barriers
        they share in the same order."""
        members, _ = self._members(ranks)
        if len(members) == 1:
            return
        mask = 0
        for r in members:
            if r != self.rank:
                self._epochs[r] = (self._epochs[r] + 1) & 0xFFFFFFFF
                mask |= 1 << r
        ep = (ctypes.c_uint * self.world)(*self._epochs)
        _lib.check(self.lib.msrl_symm_barrier(self.peer_ptrs(0), ctypes.c_int(self.rank), ctypes.c_int(self.world),
                                              ep, ctypes.c_uint(mask), _lib.ptr(self.status), _lib.stream()),
                   "symm_barrier")

    def align(self, group=None) -> None:
        """Line the ranks of ``group`` up on the current stream with a one-element library
        all-reduce.  The device barrier's wait is bounded (about two seconds); where it follows
        long, unequal work (differently packed micro-batches, rollout replicas that finish at
        different times) a healthy straggler must not run it out, so such call sites align first:
        the all-reduce has the process group's (long) timeout, and the barrier kernel behind it
        starts on every rank within microseconds of the others."""
        if self.world == 1 or not dist.is_initialized():
            return
        if getattr(self, "_align_token", None) is None:
            self._align_token = torch.zeros(1, dtype=torch.float32, device=self.device)
        dist.all_reduce(self._align_token, group=group if group is not None else self.group)

    def check(self) -> None:
        """Synchronise and raise if a barrier gave up waiting for a peer."""
        code = int(self.status.item())
        if code != 0:
            self.status.zero_()
            if 200 <= code < 300:
                raise SymmetricTimeout(f"rank {self.rank}: all-reduce timed out waiting for peer {code - 200}")
            if code >= 300:
                raise RuntimeError(f"rank {self.rank}: the expert slab of EP member {code - 300} would overflow "
                                   f"(raise moe_p2p_dispatch_rows)")
            raise SymmetricTimeout(f"rank {self.rank}: barrier timed out waiting for peer {code - 100}")

    # ---- collectives -------------------------------------------------------------------------------------
    def all_gather(self, src: torch.Tensor, dst: torch.Tensor, ranks: Optional[Sequence[int]] = None,
                   sync: bool = True) -> torch.Tensor:
        """``dst[i*n:(i+1)*n] = src on member i``; ``src`` lives in the arena at the *same offset*
        on all members, ``dst`` is any local tensor that does not overlap ``src``."""
        members, me = self._members(ranks)
        nb = src.numel() * src.element_size()
        if dst.numel() * dst.element_size() != nb * len(members):
            raise ValueError("destination must hold members x source bytes")
        off = self.offset_of(src)
        return self._gather(dst, [self.peer_base[r] + off for r in members], nb, me, ranks, sync)

    def all_gather_inplace(self, full: torch.Tensor, ranks: Optional[Sequence[int]] = None,
                           sync: bool = True) -> torch.Tensor:
        """``full`` (arena, same offset everywhere) is cut into one slice per member; member ``i``
        owns slice ``i`` of its own copy.  Afterwards every member holds all slices."""
        members, me = self._members(ranks)
        total = full.numel() * full.element_size()
        if total % (16 * len(members)):
            raise ValueError("the tensor must split into 16-byte aligned slices")
        nb = total // len(members)
        off = self.offset_of(full)
        return self._gather(full, [self.peer_base[r] + off + i * nb for i, r in enumerate(members)], nb, me,
                            ranks, sync)

    def _gather(self, dst, addresses, nb, me, ranks, sync):
        if sync:
            self.barrier(ranks)
        ptrs = (ctypes.c_void_p * len(addresses))(*addresses)
        _lib.check(self.lib.msrl_symm_all_gather(ptrs, _lib.ptr(dst), ctypes.c_longlong(nb), ctypes.c_int(me),
                                                 ctypes.c_int(len(addresses)), _lib.stream()), "symm_all_gather")
        if sync:
            self.barrier(ranks)
        return dst

    def reduce_scatter(self, src: torch.Tensor, out: Optional[torch.Tensor] = None,
                       out_f32: Optional[torch.Tensor] = None, scale: float = 1.0,
                       ranks: Optional[Sequence[int]] = None, sync: bool = True) -> None:
        """``out = scale * sum_members src[me*n:(me+1)*n]``; ``src`` (bf16 or fp32) in the arena.
        ``out`` has the dtype of ``src``; ``out_f32`` optionally receives an fp32 copy (bf16
        sources only).  ``out`` may be this rank's own slice of ``src`` (nobody else reads that
        slice); any other overlap with ``src`` is rejected because peers are reading it."""
        members, me = self._members(ranks)
        w = len(members)
        n = src.numel() // w
        if src.numel() % (w * 8):
            raise ValueError("element count must be a multiple of 8 x members")
        is_bf16 = src.dtype == torch.bfloat16
        if not is_bf16 and src.dtype != torch.float32:
            raise ValueError("reduce_scatter handles bf16 and fp32")
        lo = self.offset_of(src)
        esz = src.element_size()
        for o in (out, out_f32):
            if o is None or not self.contains(o):
                continue
            a, b = self.offset_of(o), self.offset_of(o) + o.numel() * o.element_size()
            overlaps = a < lo + src.numel() * esz and b > lo
            inside_own = lo + me * n * esz <= a and b <= lo + (me + 1) * n * esz
            if overlaps and not (inside_own and o.dtype == src.dtype):
                raise ValueError("the output may overlap the source only inside this rank's own slice")
        if sync:
            self.barrier(ranks)
        o16 = out if is_bf16 else None
        o32 = out_f32 if is_bf16 else out
        _lib.check(self.lib.msrl_symm_reduce_scatter(
            self.peer_ptrs(self.offset_of(src), members), ctypes.c_longlong(me * n), _lib.ptr(o16), _lib.ptr(o32),
            ctypes.c_longlong(n), ctypes.c_int(1 if is_bf16 else 0), ctypes.c_int(me),
            ctypes.c_int(w), ctypes.c_float(scale), _lib.stream()), "symm_reduce_scatter")
        if sync:
            self.barrier(ranks)

    def make_all_reduce(self, max_bytes: int, ranks: Optional[Sequence[int]] = None) -> "PeerAllReduce":
        """Reserve the slots of a small-message all-reduce among ``ranks`` (team positions; call on all
        members in the same order)."""
        return PeerAllReduce(self, max_bytes, ranks)

    def copy_plan(self, plan: torch.Tensor, n_desc: int, dst: torch.Tensor,
                  ranks: Optional[Sequence[int]] = None, sync: bool = True) -> None:
        """Run a resharding plan (device array of copy descriptors, see ``reshard.planner``):
        sources are arena offsets on peer ranks, destinations byte offsets into ``dst``."""
        if sync:
            self.barrier(ranks)
        _lib.check(self.lib.msrl_symm_copy_plan(self.peer_ptrs(0), _lib.ptr(dst), _lib.ptr(plan),
                                                ctypes.c_int(n_desc), ctypes.c_int(self.world), _lib.stream()),
                   "symm_copy_plan")
        if sync:
            self.barrier(ranks)

    # ---- teardown -------------------------------------------------------------------------------------------
    def close(self) -> None:
        if self._closed:
            return
        self._closed = True
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=self.group)   # nobody is still reading a peer that is about to unmap
        self._release()

    def _release(self) -> None:
        """Unmap the peers that were mapped and free the local allocation (no collective)."""
        for r, p in enumerate(self.peer_base):
            if r != self.rank and p:
                self.lib.msrl_symm_close(ctypes.c_void_p(p))
                self.peer_base[r] = 0
        self._whole = None
        if self.base:
            self.lib.msrl_symm_free(ctypes.c_void_p(self.base))
            self.base = 0
        self._closed = True


class PeerAllReduce:
    """Sum of a small bf16 tensor over a sub-team, for the two all-reduces per layer of a decode step
    under rollout tensor parallelism (reference: the row-parallel linears of the rollout engine,
    ``mindspeed_rl/models/rollout/vllm_engine.py:424-504``, all-reduce through HCCL).

    One kernel per call: every rank stores its values into its slot on every peer (posted NVLink
    stores), raises a flag there, waits for the peers' flags and adds the slots in rank order, so all
    ranks obtain bit-identical sums.  The call's sequence number lives in device memory, which makes
    the launch replayable inside a CUDA graph.  Messages larger than ``max_bytes`` are not taken
    (``fits``): bandwidth-bound sizes belong to the library collective."""

    def __init__(self, arena: "SymmetricArena", max_bytes: int, ranks: Optional[Sequence[int]] = None):
        self.arena = arena
        self.members, self.me = arena._members(ranks)
        w = len(self.members)
        self.slot_bytes = _align(int(max_bytes), 256)
        header = int(arena.lib.msrl_symm_allreduce_header_bytes())
        region = arena.alloc(header + 2 * w * self.slot_bytes, torch.uint8)
        region.zero_()
        self.region_offset = arena.offset_of(region)
        self.state = torch.zeros(int(arena.lib.msrl_symm_allreduce_state_bytes()), dtype=torch.uint8,
                                 device=arena.device)
        self._ptrs = arena.peer_ptrs(self.region_offset, self.members)
        if arena.world > 1:
            dist.barrier(group=arena.group)      # every region is zeroed before a peer may push into it

    def fits(self, t: torch.Tensor) -> bool:
        return (t.is_cuda and t.dtype == torch.bfloat16 and t.is_contiguous() and t.numel() % 8 == 0
                and t.numel() * 2 <= self.slot_bytes and t.data_ptr() % 16 == 0)

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        """In place; every member must call with the same shape in the same order."""
        if len(self.members) == 1:
            return t
        a = self.arena
        _lib.check(a.lib.msrl_symm_allreduce_push(
            self._ptrs, ctypes.c_int(self.me), ctypes.c_int(len(self.members)), _lib.ptr(t), _lib.ptr(t),
            ctypes.c_longlong(t.numel()), ctypes.c_longlong(self.slot_bytes), _lib.ptr(self.state),
            _lib.ptr(a.status), _lib.stream()), "symm_allreduce_push")
        return t


COPY_DESC_DTYPE = np.dtype([("src_off", "<i8"), ("dst_off", "<i8"), ("src_pitch", "<i8"), ("dst_pitch", "<i8"),
                            ("src_rank", "<i4"), ("rows", "<i4"), ("row_bytes", "<i4"), ("pad", "<i4")])


def plan_to_device(desc: Sequence[Tuple[int, int, int, int, int, int, int]], device) -> Tuple[torch.Tensor, int]:
    """``[(src_rank, src_off, dst_off, rows, row_bytes, src_pitch, dst_pitch)]`` -> device array."""
    arr = np.zeros(len(desc), dtype=COPY_DESC_DTYPE)
    for i, (src_rank, src_off, dst_off, rows, row_bytes, src_pitch, dst_pitch) in enumerate(desc):
        if row_bytes % 16 or src_off % 16 or dst_off % 16 or (rows > 1 and (src_pitch % 16 or dst_pitch % 16)):
            raise ValueError(f"copy descriptor {i} is not 16-byte aligned")
        arr[i] = (src_off, dst_off, src_pitch, dst_pitch, src_rank, rows, row_bytes, 0)
    t = torch.from_numpy(arr.view(np.uint8).copy())
    return t.to(device), len(desc)


_ARENA: Optional[SymmetricArena] = None


def get_arena() -> Optional[SymmetricArena]:
    return _ARENA


def init_arena(nbytes: int, group=None, device=None) -> SymmetricArena:
    """Create the process-wide arena (parameter / gradient buffers and staging live here)."""
    global _ARENA
    if _ARENA is not None:
        _ARENA.close()
    _ARENA = None
    _ARENA = SymmetricArena(nbytes, group, device)      # ArenaUnavailable leaves no arena behind
    return _ARENA
