"""Megatron-compatible indexed datasets (``<prefix>.bin`` token data + ``<prefix>.idx`` index).

Index layout (little endian): 9-byte magic ``MMIDIDX\\0\\0``, ``uint64`` version (1), ``uint8``
dtype code, ``uint64`` sequence count, ``uint64`` document count, ``int32[seq]`` lengths,
``int64[seq]`` byte pointers, ``int64[doc]`` document boundaries, and for multimodal data an
``int8[seq]`` mode vector.  A tokenised RL / SFT dataset is a set of such files named
``{prefix}_packed_{field}_document.{bin,idx}`` (``input_ids``, ``labels``, ``attention_mask``, ...),
exposed together by :class:`CombinedDataset`.  Files written here can be read by Megatron-style
tooling and vice versa (reference reader/writer: ``mindspeed_rl/datasets/indexed_dataset.py``).
"""
from __future__ import annotations

import glob
import os
import re
import struct
from typing import Dict, Iterable, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

MAGIC = b"MMIDIDX\x00\x00"
_CODES = {1: np.uint8, 2: np.int8, 3: np.int16, 4: np.int32, 5: np.int64, 6: np.float64, 7: np.float32,
          8: np.uint16}
_BY_DTYPE = {np.dtype(v): k for k, v in _CODES.items()}


def dtype_code(dtype) -> int:
    return _BY_DTYPE[np.dtype(dtype)]


def optimal_dtype(cardinality: Optional[int]):
    """Smallest integer type that can hold token ids below ``cardinality``."""
    return np.uint16 if cardinality is not None and cardinality < 65500 else np.int32


def get_idx_path(prefix: str) -> str:
    return prefix + ".idx"


def get_bin_path(prefix: str) -> str:
    return prefix + ".bin"


class _Index:
    def __init__(self, path: str, multimodal: bool = False):
        with open(path, "rb") as fh:
            if fh.read(9) != MAGIC:
                raise ValueError(f"{path}: not an MMIDIDX index file")
            (version,) = struct.unpack("<Q", fh.read(8))
            if version != 1:
                raise ValueError(f"{path}: unsupported index version {version}")
            (code,) = struct.unpack("<B", fh.read(1))
            self.dtype = np.dtype(_CODES[code])
            (self.sequence_count,) = struct.unpack("<Q", fh.read(8))
            (self.document_count,) = struct.unpack("<Q", fh.read(8))
            offset = fh.tell()
        self._mmap = np.memmap(path, mode="r", order="C")
        n, d = self.sequence_count, self.document_count
        self.lengths = np.frombuffer(self._mmap, dtype=np.int32, count=n, offset=offset)
        offset += 4 * n
        self.pointers = np.frombuffer(self._mmap, dtype=np.int64, count=n, offset=offset)
        offset += 8 * n
        self.doc_idx = np.frombuffer(self._mmap, dtype=np.int64, count=d, offset=offset)
        offset += 8 * d
        self.modes = np.frombuffer(self._mmap, dtype=np.int8, count=n, offset=offset) if multimodal else None


class IndexedDataset(torch.utils.data.Dataset):
    """Random access to the sequences of one ``.bin/.idx`` pair (memory mapped)."""

    def __init__(self, path_prefix: str, multimodal: bool = False, mmap: bool = True,
                 max_len: Optional[int] = None):
        self.path_prefix, self.multimodal, self.max_len = path_prefix, multimodal, max_len
        self.index = _Index(get_idx_path(path_prefix), multimodal)
        self._bin = np.memmap(get_bin_path(path_prefix), mode="r", order="C") if mmap else \
            np.fromfile(get_bin_path(path_prefix), dtype=np.uint8)
        self._keep = np.arange(self.index.sequence_count)
        self._doc_idx = self.index.doc_idx

    def __len__(self) -> int:
        return len(self._keep)

    def _read(self, seq: int, offset: int = 0, length: Optional[int] = None) -> np.ndarray:
        n = int(self.index.lengths[seq])
        length = n - offset if length is None else length
        start = int(self.index.pointers[seq]) + offset * self.index.dtype.itemsize
        return np.frombuffer(self._bin, dtype=self.index.dtype, count=length, offset=start)

    def __getitem__(self, idx: Union[int, np.integer, slice]):
        if isinstance(idx, slice):
            return [self[i] for i in range(*idx.indices(len(self)))]
        seq = int(self._keep[idx])
        data = self._read(seq)
        return (data, self.index.modes[seq]) if self.index.modes is not None else data

    def get(self, idx: int, offset: int = 0, length: Optional[int] = None) -> np.ndarray:
        return self._read(int(self._keep[idx]), offset, length)

    def get_filter_mask(self) -> np.ndarray:
        if self.max_len is None:
            return np.ones(len(self), dtype=bool)
        return self.index.lengths[self._keep] <= self.max_len

    def do_filter(self, mask: np.ndarray) -> None:
        self._keep = self._keep[np.asarray(mask, dtype=bool)]

    @property
    def sequence_lengths(self) -> np.ndarray:
        return self.index.lengths[self._keep]

    @property
    def document_indices(self) -> np.ndarray:
        return self._doc_idx

    def get_document_indices(self) -> np.ndarray:
        return self._doc_idx

    def set_document_indices(self, doc_idx: np.ndarray) -> None:
        self._doc_idx = doc_idx

    @property
    def sequence_modes(self):
        return self.index.modes

    @staticmethod
    def exists(path_prefix: str) -> bool:
        return os.path.exists(get_idx_path(path_prefix)) and os.path.exists(get_bin_path(path_prefix))


class CombinedDataset(torch.utils.data.Dataset):
    """Several aligned field datasets read together: ``ds[i] -> {field: array}``."""

    def __init__(self, datasets: Dict[str, IndexedDataset]):
        sizes = {len(d) for d in datasets.values()}
        if len(sizes) > 1:
            raise ValueError(f"field datasets differ in length: { {k: len(v) for k, v in datasets.items()} }")
        self.datasets = datasets

    def __len__(self) -> int:
        return len(next(iter(self.datasets.values()))) if self.datasets else 0

    def __getitem__(self, idx):
        return {k: d[idx] for k, d in self.datasets.items()}


def get_packed_indexed_dataset(data_prefix: str, filter_length: Optional[int] = None,
                               is_pairwise_dataset: bool = False) -> CombinedDataset:
    """Open every ``{prefix}_packed_{field}_document`` pair; optionally drop samples whose
    ``input_ids`` exceed ``filter_length`` (all fields are filtered consistently)."""
    fields = set()
    for name in glob.glob(f"{data_prefix}_packed_*_document*"):
        m = re.match(re.escape(data_prefix) + r"_packed_(.*)_document(.*)", name)
        if m:
            fields.add(m.group(1))
    if not fields:
        raise FileNotFoundError(f"no packed dataset files found for prefix '{data_prefix}'")
    ds = {f: IndexedDataset(f"{data_prefix}_packed_{f}_document",
                            max_len=filter_length if (filter_length and f == "input_ids") else None)
          for f in sorted(fields)}
    if filter_length and not is_pairwise_dataset and "input_ids" in ds:
        mask = ds["input_ids"].get_filter_mask()
        for d in ds.values():
            d.do_filter(mask)
    return CombinedDataset(ds)


class IndexedDatasetBuilder:
    """Streams sequences into a ``.bin`` file and writes the matching ``.idx`` at ``finalize``."""

    def __init__(self, bin_path: str, dtype=np.int32, multimodal: bool = False, buffer_items: int = 1 << 16):
        self._fh = open(bin_path, "wb")
        self.dtype = np.dtype(dtype)
        self.multimodal = multimodal
        self.lengths: List[int] = []
        self.doc_idx: List[int] = [0]
        self.modes: Optional[List[int]] = [] if multimodal else None
        self._buf: List[np.ndarray] = []
        self._buffered = 0
        self._limit = buffer_items

    def _flush(self) -> None:
        if self._buf:
            self._fh.write(np.concatenate(self._buf).tobytes(order="C"))
            self._buf, self._buffered = [], 0

    def add_item(self, tensor, mode: int = 0) -> None:
        arr = np.asarray(tensor.numpy() if torch.is_tensor(tensor) else tensor, dtype=self.dtype).reshape(-1)
        self._buf.append(arr)
        self._buffered += arr.size
        self.lengths.append(arr.size)
        if self.modes is not None:
            self.modes.append(mode)
        if self._buffered >= self._limit:
            self._flush()

    def add_document(self, tensor, lengths: Sequence[int], modes: Optional[Sequence[int]] = None) -> None:
        arr = np.asarray(tensor.numpy() if torch.is_tensor(tensor) else tensor, dtype=self.dtype).reshape(-1)
        self._buf.append(arr)
        self._buffered += arr.size
        self.lengths.extend(int(x) for x in lengths)
        if self.modes is not None:
            self.modes.extend(modes if modes is not None else [0] * len(lengths))
        self.end_document()
        if self._buffered >= self._limit:
            self._flush()

    def end_document(self) -> None:
        self.doc_idx.append(len(self.lengths))

    def add_index(self, path_prefix: str) -> None:
        """Append another dataset (used when merging the shards of parallel preprocessing)."""
        other = _Index(get_idx_path(path_prefix), self.multimodal)
        if other.dtype != self.dtype:
            raise ValueError("cannot merge datasets of different dtypes")
        self._flush()
        base = len(self.lengths)
        self.lengths.extend(other.lengths.tolist())
        self.doc_idx.extend((base + other.doc_idx[1:]).tolist())
        if self.modes is not None and other.modes is not None:
            self.modes.extend(other.modes.tolist())
        with open(get_bin_path(path_prefix), "rb") as src:
            while True:
                chunk = src.read(1 << 24)
                if not chunk:
                    break
                self._fh.write(chunk)

    def finalize(self, idx_path: str) -> None:
        self._flush()
        self._fh.close()
        lengths = np.asarray(self.lengths, dtype=np.int32)
        pointers = np.zeros(len(lengths), dtype=np.int64)
        if len(lengths) > 1:
            np.cumsum(lengths[:-1].astype(np.int64) * self.dtype.itemsize, out=pointers[1:])
        with open(idx_path, "wb") as fh:
            fh.write(MAGIC)
            fh.write(struct.pack("<Q", 1))
            fh.write(struct.pack("<B", dtype_code(self.dtype)))
            fh.write(struct.pack("<Q", len(lengths)))
            fh.write(struct.pack("<Q", len(self.doc_idx)))
            fh.write(lengths.tobytes(order="C"))
            fh.write(pointers.tobytes(order="C"))
            fh.write(np.asarray(self.doc_idx, dtype=np.int64).tobytes(order="C"))
            if self.modes is not None:
                fh.write(np.asarray(self.modes, dtype=np.int8).tobytes(order="C"))
