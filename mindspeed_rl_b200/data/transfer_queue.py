"""TransferQueue: the sharded experience store (control plane / data plane split).

The single-process ``TransferDock`` moves every tensor through one Python object.  The queue
splits that role (reference: ``mindspeed_rl/utils/transfer_queue/tq_mgr.py:24-1080``,
``tq_data.py:22-283``, ``tq_client.py:31-545``, ``tq_utils.py:335-430``,
``trainer/utils/data_strategy.py:74-850``):

* ``TransferQueueManager`` keeps only metadata -- ready bits, per-consumer consumption, ages and
  partial-rollout state, metrics -- and answers "which rows may this consumer take";
* ``TransferQueueShard``s hold the tensors (row ``i`` lives on shard ``i % num_shards``), each
  behind its own ZeroMQ ROUTER socket speaking ``PUT`` / ``GET`` / ``CLEAR`` with a small pickled
  header and a raw binary tensor-list payload (dtype / shape table + concatenated bytes, no
  per-tensor pickling);
* ``TransferQueueClient`` talks to all shards in parallel over thread-local DEALER sockets;
* ``SyncTransferQueueAdapter`` gives the pair the ``TransferDock`` API the workers and trainers
  use, so ``DataStrategy`` can switch between ``td`` and ``tq`` by name.
"""
from __future__ import annotations

import pickle
import queue
import struct
import threading
import time
from typing import Any, Dict, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch
import zmq

from ..utils.pad_process import padding_dict_to_tensor_dict, remove_padding_tensor_dict_to_dict
from .transfer_dock import GRPOTransferDock, trans_input_to_experience

# ---- binary tensor-list codec -----------------------------------------------------------------------
_DTYPES = [torch.float32, torch.float16, torch.bfloat16, torch.int64, torch.int32, torch.int16, torch.int8,
           torch.uint8, torch.bool, torch.float64]
_DTYPE_CODE = {d: i for i, d in enumerate(_DTYPES)}


def encode_tensor_list(tensors: Sequence[Optional[torch.Tensor]]) -> bytes:
    """``[count][per tensor: dtype u8, ndim u8, dims i64...][payload]``; ``None`` -> dtype 255."""
    head = [struct.pack("<I", len(tensors))]
    body = []
    for t in tensors:
        if t is None:
            head.append(struct.pack("<BB", 255, 0))
            continue
        t = t.detach().cpu().contiguous()
        head.append(struct.pack("<BB", _DTYPE_CODE[t.dtype], t.dim()) + struct.pack(f"<{t.dim()}q", *t.shape))
        flat = t.reshape(-1)
        body.append(flat.view(torch.uint8).numpy().tobytes() if t.dtype != torch.bool
                    else flat.to(torch.uint8).numpy().tobytes())
    return b"".join(head) + b"".join(body)


def decode_tensor_list(buf: bytes) -> List[Optional[torch.Tensor]]:
    (count,) = struct.unpack_from("<I", buf, 0)
    off = 4
    metas = []
    for _ in range(count):
        code, ndim = struct.unpack_from("<BB", buf, off)
        off += 2
        shape = struct.unpack_from(f"<{ndim}q", buf, off) if ndim else ()
        off += 8 * ndim
        metas.append((code, tuple(shape)))
    out: List[Optional[torch.Tensor]] = []
    for code, shape in metas:
        if code == 255:
            out.append(None)
            continue
        dtype = _DTYPES[code]
        esz = 1 if dtype == torch.bool else torch.empty(0, dtype=dtype).element_size()
        n = int(np.prod(shape)) if shape else 1
        if n == 0:
            out.append(torch.empty(shape, dtype=dtype))
            continue
        raw = torch.frombuffer(bytearray(buf[off:off + n * esz]), dtype=torch.uint8)
        off += n * esz
        t = raw.to(torch.bool) if dtype == torch.bool else raw.view(dtype)
        out.append(t.reshape(shape))
    return out


# ---- data plane -------------------------------------------------------------------------------------------
class TransferQueueShard:
    """Tensor storage of the rows ``i`` with ``i % num_shards == shard_id`` plus its ROUTER server."""

    def __init__(self, shard_id: int, num_shards: int, bind: str = "tcp://127.0.0.1:0", timeout_s: float = 300.0):
        self.shard_id, self.num_shards, self.timeout_s = shard_id, num_shards, timeout_s
        self.rows: Dict[str, Dict[int, torch.Tensor]] = {}
        self._cv = threading.Condition()
        self.ctx = zmq.Context.instance()
        self.sock = self.ctx.socket(zmq.ROUTER)
        port = self.sock.bind_to_random_port(bind[:-2]) if bind.endswith(":0") else None
        if port is None:
            self.sock.bind(bind)
        self.address = f"{bind[:-2]}:{port}" if port is not None else bind
        self._stop = threading.Event()
        self._replies: "queue.Queue" = queue.Queue()
        self._thread = threading.Thread(target=self._serve, daemon=True)
        self._thread.start()

    # storage ------------------------------------------------------------------------------------
    def put(self, columns: Sequence[str], indexes: Sequence[int], tensors: Sequence[torch.Tensor]) -> None:
        with self._cv:
            k = 0
            for c in columns:
                col = self.rows.setdefault(c, {})
                for i in indexes:
                    col[i] = tensors[k]
                    k += 1
            self._cv.notify_all()

    def get(self, columns: Sequence[str], indexes: Sequence[int]) -> List[torch.Tensor]:
        deadline = time.time() + self.timeout_s
        with self._cv:
            while not all(i in self.rows.get(c, {}) for c in columns for i in indexes):
                left = deadline - time.time()
                if left <= 0:
                    raise TimeoutError(f"shard {self.shard_id}: rows never arrived for columns {list(columns)}")
                self._cv.wait(min(left, 0.5))
            return [self.rows[c][i] for c in columns for i in indexes]

    def clear(self, indexes: Optional[Sequence[int]] = None) -> None:
        with self._cv:
            if indexes is None:
                self.rows.clear()
            else:
                for col in self.rows.values():
                    for i in indexes:
                        col.pop(i, None)

    # server -------------------------------------------------------------------------------------
    def _serve(self) -> None:
        # Only this thread touches the socket: handler threads (a GET may block until its rows
        # arrive) hand their replies back through a queue.
        poller = zmq.Poller()
        poller.register(self.sock, zmq.POLLIN)
        pending = 0
        while not self._stop.is_set():
            try:
                if dict(poller.poll(1 if pending else 50)):
                    ident, header, payload = self.sock.recv_multipart()
                    pending += 1
                    threading.Thread(target=self._handle, args=(ident, header, payload), daemon=True).start()
                while not self._replies.empty():
                    self.sock.send_multipart(self._replies.get_nowait())
                    pending -= 1
            except zmq.ZMQError:
                break
        self.sock.close(0)

    def _handle(self, ident: bytes, header: bytes, payload: bytes) -> None:
        try:
            h = pickle.loads(header)
            if h["op"] == "PUT":
                self.put(h["columns"], h["indexes"], decode_tensor_list(payload))
                reply = (pickle.dumps({"ok": True}), b"")
            elif h["op"] == "GET":
                reply = (pickle.dumps({"ok": True}), encode_tensor_list(self.get(h["columns"], h["indexes"])))
            elif h["op"] == "CLEAR":
                self.clear(h.get("indexes"))
                reply = (pickle.dumps({"ok": True}), b"")
            else:
                raise ValueError(f"unknown op {h['op']}")
        except Exception as e:  # the error travels back to the caller
            reply = (pickle.dumps({"ok": False, "error": f"{type(e).__name__}: {e}"}), b"")
        self._replies.put([ident, *reply])

    def shutdown(self) -> None:
        self._stop.set()


class TransferQueueClient:
    def __init__(self, shard_addresses: Sequence[str], timeout_s: float = 600.0):
        self.addresses = list(shard_addresses)
        self.timeout_ms = int(timeout_s * 1000)
        self._local = threading.local()

    def _socks(self):
        socks = getattr(self._local, "socks", None)
        if socks is None:
            ctx = zmq.Context.instance()
            socks = []
            for a in self.addresses:
                s = ctx.socket(zmq.DEALER)
                s.setsockopt(zmq.LINGER, 0)
                s.connect(a)
                socks.append(s)
            self._local.socks = socks
        return socks

    def _round_trip(self, requests: Dict[int, Tuple[dict, bytes]]) -> Dict[int, bytes]:
        socks = self._socks()
        for shard, (header, payload) in requests.items():
            socks[shard].send_multipart([pickle.dumps(header), payload])
        out = {}
        for shard in requests:
            if not socks[shard].poll(self.timeout_ms):
                raise TimeoutError(f"transfer-queue shard {shard} did not answer")
            header, payload = socks[shard].recv_multipart()
            h = pickle.loads(header)
            if not h.get("ok"):
                raise RuntimeError(f"transfer-queue shard {shard}: {h.get('error')}")
            out[shard] = payload
        return out

    def _partition(self, indexes: Sequence[int]) -> Dict[int, List[int]]:
        parts: Dict[int, List[int]] = {}
        for pos, idx in enumerate(indexes):
            parts.setdefault(idx % len(self.addresses), []).append(pos)
        return parts

    def put(self, data: Dict[str, List[torch.Tensor]], indexes: Sequence[int]) -> None:
        columns = list(data)
        reqs = {}
        for shard, positions in self._partition(indexes).items():
            tensors = [data[c][p] for c in columns for p in positions]
            reqs[shard] = ({"op": "PUT", "columns": columns, "indexes": [indexes[p] for p in positions]},
                           encode_tensor_list(tensors))
        self._round_trip(reqs)

    def get(self, columns: Sequence[str], indexes: Sequence[int]) -> Dict[str, List[torch.Tensor]]:
        parts = self._partition(indexes)
        reqs = {s: ({"op": "GET", "columns": list(columns), "indexes": [indexes[p] for p in pos]}, b"")
                for s, pos in parts.items()}
        replies = self._round_trip(reqs)
        out: Dict[str, List[Optional[torch.Tensor]]] = {c: [None] * len(indexes) for c in columns}
        for shard, positions in parts.items():
            tensors = decode_tensor_list(replies[shard])
            k = 0
            for c in columns:
                for p in positions:
                    out[c][p] = tensors[k]
                    k += 1
        return out

    def clear(self, indexes: Optional[Sequence[int]] = None) -> None:
        self._round_trip({s: ({"op": "CLEAR", "indexes": None if indexes is None else
                               [i for i in indexes if i % len(self.addresses) == s]}, b"")
                          for s in range(len(self.addresses))})


# ---- control plane ------------------------------------------------------------------------------------------
class TransferQueueManager(GRPOTransferDock):
    """Metadata-only dock: rows are registered with one-byte-per-element placeholders (so that
    ready bits, sequence-length balancing, ages and partial-rollout bookkeeping behave exactly as
    in the single-process dock), the tensors themselves live on the shards."""

    def register_put(self, lengths: Dict[str, List[int]], indexes: List[int], is_prompt: bool = False,
                     rollout_completed: Optional[List[int]] = None) -> None:
        data: Dict[str, List[torch.Tensor]] = {
            c: [torch.zeros(max(int(n), 1), dtype=torch.int8) for n in ls] for c, ls in lengths.items()}
        if rollout_completed is not None:
            data["rollout_completed"] = [torch.tensor([int(f)], dtype=torch.int32) for f in rollout_completed]
        super().put_experience(padding_dict_to_tensor_dict(data), indexes, is_prompt=is_prompt)

    def is_partial_rollout(self) -> bool:
        return bool(self.enable_partial_rollout)

    def sample(self, consumer: str, columns: List[str], experience_count: Optional[int] = None, dp_size: int = 1,
               indexes: Optional[List[int]] = None, get_n_samples: bool = True,
               use_batch_seqlen_balance: bool = False):
        """Row indexes ``consumer`` may read now (marks them consumed) and their ages when asked."""
        batch, idx = super().get_experience(consumer, columns, experience_count, dp_size, indexes, get_n_samples,
                                            use_batch_seqlen_balance)
        if idx is None:
            return None, None
        return idx, (batch["age"] if "age" in columns else None)


class SyncTransferQueueAdapter:
    """``TransferDock``-shaped facade over a manager handle (local object or RPC proxy) and a
    shard client."""

    def __init__(self, manager, client: TransferQueueClient):
        self.manager, self.client = manager, client

    def get_experience(self, consumer: str, experience_columns: List[str], experience_count: Optional[int] = None,
                       dp_size: int = 1, indexes: Optional[List[int]] = None, get_n_samples: bool = True,
                       use_batch_seqlen_balance: bool = False, allow_partial_ready_data: bool = False):
        idx, age = self.manager.sample(consumer, list(experience_columns), experience_count, dp_size, indexes,
                                       get_n_samples, use_batch_seqlen_balance)
        if not idx:
            return None, None
        columns = [c for c in experience_columns if c != "age"]
        real = [i for i in idx if i >= 0]
        rows = self.client.get(columns, real)
        if len(real) < len(idx):                      # filler rows (-2) repeat the last real row
            for c in columns:
                rows[c] = rows[c] + [rows[c][-1]] * (len(idx) - len(real))
        batch = padding_dict_to_tensor_dict(rows)
        if age is not None:
            batch["age"] = age
        return batch, idx

    def put_experience(self, data_dict: Dict[str, Union[torch.Tensor, List[torch.Tensor]]],
                       indexes: Optional[List[int]] = None, is_prompt: bool = False) -> None:
        if not indexes:
            raise ValueError("put_experience needs the row indexes")
        names, cols = trans_input_to_experience(remove_padding_tensor_dict_to_dict(data_dict))
        data = dict(zip(names, cols))
        completed = None
        if "rollout_completed" in data:
            completed = [int(t.reshape(-1)[0]) for t in data.pop("rollout_completed")]
        keep = [p for p, i in enumerate(indexes) if i >= 0]
        real_idx = [indexes[p] for p in keep]
        narrowed = {c: [GRPOTransferDock._narrow(rows[p]) for p in keep] for c, rows in data.items()}
        if is_prompt and self.manager.is_partial_rollout():
            # fresh prompts start with an empty response that the rollout stage will continue
            narrowed["responses"] = [torch.tensor([-1], dtype=torch.int32) for _ in real_idx]
            narrowed["response_length"] = [torch.tensor([0], dtype=torch.int32) for _ in real_idx]
        self.client.put(narrowed, real_idx)           # data first, then the ready bits
        narrowed = {c: r for c, r in narrowed.items() if not (is_prompt and c in ("responses", "response_length")
                                                              and c not in data)}
        self.manager.register_put({c: [t.numel() for t in rows] for c, rows in narrowed.items()}, real_idx,
                                  is_prompt, None if completed is None else [completed[p] for p in keep])

    def clear(self, consumer: str = "actor_train") -> None:
        self.manager.clear(consumer)
        self.client.clear(None)

    def __getattr__(self, name: str):                 # all_consumed, metrics, partial-rollout state, ...
        return getattr(self.manager, name)


# ---- strategy ---------------------------------------------------------------------------------------------------
_ALIASES = {"td": "td", "transfer_dock": "td", "transferdock": "td", "dock": "td",
            "tq": "tq", "transfer_queue": "tq", "transferqueue": "tq", "queue": "tq"}


class DataStrategy:
    """Builds the experience store named by ``rl_config.data_strategy`` (``td`` default, ``tq``)."""

    def __init__(self, kind: str = "td", num_shards: int = 2):
        key = _ALIASES.get(str(kind or "td").lower())
        if key is None:
            raise ValueError(f"unknown data strategy '{kind}' (known: {sorted(set(_ALIASES))})")
        self.kind, self.num_shards = key, max(int(num_shards), 1)
        self.shards: List[TransferQueueShard] = []

    def create(self, *args, **kwargs):
        """Driver side: ``(store object to serve or use, descriptor to broadcast)``."""
        if self.kind == "td":
            return GRPOTransferDock(*args, **kwargs), None
        manager = TransferQueueManager(*args, **kwargs)
        self.shards = [TransferQueueShard(i, self.num_shards) for i in range(self.num_shards)]
        return manager, {"shards": [s.address for s in self.shards]}

    @staticmethod
    def attach(handle, descriptor):
        """Any rank: wrap the (possibly remote) manager handle for use."""
        if not descriptor:
            return handle
        return SyncTransferQueueAdapter(handle, TransferQueueClient(descriptor["shards"]))
