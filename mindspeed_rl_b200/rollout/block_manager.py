"""ctypes front-end of the C++ paged-KV block manager (``csrc/block_manager.cpp``)."""
from __future__ import annotations

import ctypes
from pathlib import Path
from typing import List, Optional, Sequence, Tuple

import numpy as np

_HOST_LIB = Path(__file__).resolve().parent.parent / "_C" / "libmsrl_host.so"
_lib: Optional[ctypes.CDLL] = None


def _load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not _HOST_LIB.exists():
            from ..csrc import build

            build.build()
        L = ctypes.CDLL(str(_HOST_LIB))
        L.msrl_bm_create.restype = ctypes.c_void_p
        L.msrl_bm_create.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int]
        L.msrl_bm_destroy.argtypes = [ctypes.c_void_p]
        L.msrl_bm_num_free.argtypes = [ctypes.c_void_p]
        L.msrl_bm_blocks_needed.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64]
        L.msrl_bm_allocate.restype = ctypes.c_int64
        L.msrl_bm_allocate.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64]
        L.msrl_bm_append.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64]
        L.msrl_bm_commit.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64]
        L.msrl_bm_fork.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p]
        L.msrl_bm_free.argtypes = [ctypes.c_void_p, ctypes.c_int64]
        L.msrl_bm_num_blocks.argtypes = [ctypes.c_void_p, ctypes.c_int64]
        L.msrl_bm_block_table.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int]
        L.msrl_bm_block_tables.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                                           ctypes.c_void_p, ctypes.c_int]
        L.msrl_bm_slots.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                    ctypes.c_void_p]
        L.msrl_bm_stats.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        _lib = L
    return _lib


class OutOfBlocks(RuntimeError):
    pass


class BlockManager:
    """Physical-block bookkeeping of the paged KV cache (allocation, sharing, prefix cache)."""

    def __init__(self, num_blocks: int, block_size: int, enable_prefix_caching: bool = False):
        self._L = _load()
        self.num_blocks, self.block_size = num_blocks, block_size
        self.enable_prefix_caching = enable_prefix_caching
        self._h = self._L.msrl_bm_create(num_blocks, block_size, 1 if enable_prefix_caching else 0)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._L.msrl_bm_destroy(h)

    @property
    def num_free_blocks(self) -> int:
        return self._L.msrl_bm_num_free(self._h)

    def blocks_needed(self, seq_id: int, new_total_tokens: int) -> int:
        return self._L.msrl_bm_blocks_needed(self._h, seq_id, new_total_tokens)

    def allocate(self, seq_id: int, tokens: Sequence[int]) -> int:
        """Reserve blocks for a prompt; returns the number of leading tokens found in the prefix
        cache.  Raises :class:`OutOfBlocks` when the prompt does not fit right now."""
        arr = np.ascontiguousarray(tokens, dtype=np.int32)
        r = self._L.msrl_bm_allocate(self._h, seq_id, arr.ctypes.data, arr.size)
        if r == -1:
            raise OutOfBlocks()
        if r < 0:
            raise KeyError(f"sequence {seq_id} already allocated")
        return int(r)

    def can_append(self, n_seqs: int = 1) -> bool:
        return self.num_free_blocks >= n_seqs

    def append(self, seq_id: int, n_new: int = 1) -> None:
        r = self._L.msrl_bm_append(self._h, seq_id, n_new)
        if r == -1:
            raise OutOfBlocks()
        if r < 0:
            raise KeyError(seq_id)

    def commit(self, seq_id: int, tokens: Sequence[int], n_computed: int) -> None:
        if not self.enable_prefix_caching:
            return
        arr = np.ascontiguousarray(tokens, dtype=np.int32)
        self._L.msrl_bm_commit(self._h, seq_id, arr.ctypes.data, int(n_computed))

    def fork(self, parent_id: int, child_id: int) -> Tuple[int, int]:
        """Child shares the parent's full blocks; returns (src, dst) of the partial block to copy
        (``(-1, -1)`` when there is none)."""
        pair = (ctypes.c_int32 * 2)()
        r = self._L.msrl_bm_fork(self._h, parent_id, child_id, pair)
        if r == -1:
            raise OutOfBlocks()
        if r < 0:
            raise KeyError((parent_id, child_id))
        return int(pair[0]), int(pair[1])

    def free(self, seq_id: int) -> None:
        self._L.msrl_bm_free(self._h, seq_id)

    def block_table(self, seq_id: int) -> List[int]:
        n = self._L.msrl_bm_num_blocks(self._h, seq_id)
        if n < 0:
            raise KeyError(seq_id)
        out = np.zeros(max(n, 1), dtype=np.int32)
        self._L.msrl_bm_block_table(self._h, seq_id, out.ctypes.data, n)
        return out[:n].tolist()

    def block_tables(self, seq_ids: Sequence[int], max_blocks: int, out: Optional[np.ndarray] = None
                     ) -> np.ndarray:
        ids = np.ascontiguousarray(seq_ids, dtype=np.int64)
        if out is None:
            out = np.zeros((len(ids), max_blocks), dtype=np.int32)
        r = self._L.msrl_bm_block_tables(self._h, ids.ctypes.data, len(ids), out.ctypes.data, max_blocks)
        if r != 0:
            raise RuntimeError(f"block_tables failed ({r})")
        return out

    def slots(self, seq_id: int, start: int, count: int) -> np.ndarray:
        out = np.empty(count, dtype=np.int64)
        r = self._L.msrl_bm_slots(self._h, seq_id, start, count, out.ctypes.data)
        if r != 0:
            raise RuntimeError(f"slots failed ({r}) for seq {seq_id} [{start}, {start + count})")
        return out

    def stats(self) -> dict:
        out = (ctypes.c_int64 * 4)()
        self._L.msrl_bm_stats(self._h, out)
        return {"free_blocks": out[0], "sequences": out[1], "prefix_hits": out[2],
                "prefix_queries": out[3]}
