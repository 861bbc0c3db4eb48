"""Reliable one-to-many fan-out of small host messages inside a model replica over ZeroMQ.

The leader of a replica (tp 0, cp 0, pp 0) pulls a batch from the experience store and must hand
the same batch to the other ranks of its replica.  For payloads under ``threshold_bytes`` a
PUB/SUB socket with acknowledgements is cheaper than a collective on the accelerator stream and
does not serialise with in-flight kernels (reference: ``mindspeed_rl/utils/zmq_communication.py:
49-440``, used by ``workers/base_worker.py:518-682`` for batches below 10 MB):

* server: ``PUB`` (data), ``REP`` (registration), ``PULL`` (acks); every message carries a sequence
  number; the server re-publishes until all registered clients have acknowledged it (every
  ``resend_interval`` seconds) and raises ``TimeoutError`` after ``max_resends`` rounds;
* client: registers once (REQ), subscribes, returns messages strictly in sequence order,
  drops duplicates and acknowledges what it has delivered.

The server address reaches the clients through one ``broadcast_object_list`` over the replica's
process group at start-up (``setup_replica_broadcast``).
"""
from __future__ import annotations

import pickle
import socket
import threading
import time
import uuid
from typing import Any, Dict, Optional, Set

import zmq


def _free_port(host: str = "127.0.0.1") -> int:
    with socket.socket() as s:
        s.bind((host, 0))
        return s.getsockname()[1]


class ZmqServer:
    def __init__(self, num_clients: int, host: str = "127.0.0.1", resend_interval: float = 1.0,
                 max_resends: int = 60):
        self.num_clients, self.resend_interval, self.max_resends = num_clients, resend_interval, max_resends
        self.ctx = zmq.Context.instance()
        self.pub, self.rep, self.pull = (self.ctx.socket(t) for t in (zmq.PUB, zmq.REP, zmq.PULL))
        ports = []
        for sock in (self.pub, self.rep, self.pull):
            sock.setsockopt(zmq.LINGER, 0)
            ports.append(sock.bind_to_random_port(f"tcp://{host}"))
        self.address = dict(host=host, pub=ports[0], rep=ports[1], pull=ports[2])
        self.clients: Set[str] = set()
        self.seq = 0

    def wait_for_clients(self, timeout: float = 60.0) -> None:
        """Serve registration requests until ``num_clients`` distinct clients are known."""
        deadline = time.time() + timeout
        while len(self.clients) < self.num_clients:
            left = deadline - time.time()
            if left <= 0:
                raise TimeoutError(f"only {len(self.clients)} of {self.num_clients} clients registered")
            if self.rep.poll(int(min(left, 0.2) * 1000)):
                cid = self.rep.recv_string()
                self.clients.add(cid)
                self.rep.send_string("ok")

    def broadcast(self, obj: Any) -> int:
        """Publish ``obj`` and return once every client has acknowledged it."""
        if len(self.clients) < self.num_clients:
            self.wait_for_clients()
        self.seq += 1
        frame = [str(self.seq).encode(), pickle.dumps(obj, protocol=pickle.HIGHEST_PROTOCOL)]
        pending = set(self.clients)
        wait = min(0.05, self.resend_interval)         # early re-sends cover a subscriber that joined late
        for _ in range(self.max_resends + 5):
            self.pub.send_multipart(frame)
            deadline = time.time() + wait
            wait = min(wait * 2, self.resend_interval)
            while pending and time.time() < deadline:
                if self.pull.poll(int(max(deadline - time.time(), 0) * 1000)):
                    cid, seq = self.pull.recv_multipart()
                    if int(seq) == self.seq:
                        pending.discard(cid.decode())
            if not pending:
                return self.seq
        raise TimeoutError(f"message {self.seq}: no acknowledgement from {sorted(pending)} after "
                           f"{self.max_resends} resends")

    def close(self) -> None:
        for s in (self.pub, self.rep, self.pull):
            s.close(0)


class ZmqClient:
    def __init__(self, address: Dict[str, Any], client_id: Optional[str] = None, register_timeout: float = 60.0):
        self.id = client_id or uuid.uuid4().hex
        self.ctx = zmq.Context.instance()
        host = address["host"]
        self.sub, self.push = self.ctx.socket(zmq.SUB), self.ctx.socket(zmq.PUSH)
        for s in (self.sub, self.push):
            s.setsockopt(zmq.LINGER, 0)
        self.sub.setsockopt(zmq.SUBSCRIBE, b"")
        self.sub.connect(f"tcp://{host}:{address['pub']}")
        self.push.connect(f"tcp://{host}:{address['pull']}")
        req = self.ctx.socket(zmq.REQ)
        req.setsockopt(zmq.LINGER, 0)
        req.connect(f"tcp://{host}:{address['rep']}")
        req.send_string(self.id)
        if not req.poll(int(register_timeout * 1000)):
            req.close(0)
            raise TimeoutError("the broadcast server did not answer the registration")
        req.recv_string()
        req.close(0)
        self.next_seq = 1

    def receive(self, timeout: float = 120.0) -> Any:
        """Next message in sequence order (duplicates from re-sends are acknowledged and dropped)."""
        deadline = time.time() + timeout
        while True:
            left = deadline - time.time()
            if left <= 0:
                raise TimeoutError(f"client {self.id}: message {self.next_seq} never arrived")
            if not self.sub.poll(int(min(left, 0.5) * 1000)):
                continue
            seq_b, payload = self.sub.recv_multipart()
            seq = int(seq_b)
            self.push.send_multipart([self.id.encode(), seq_b])
            if seq == self.next_seq:
                self.next_seq += 1
                return pickle.loads(payload)
            # seq < next_seq: a re-send of something already delivered; seq > next_seq cannot
            # happen because the server waits for all acknowledgements before the next message

    def close(self) -> None:
        self.sub.close(0)
        self.push.close(0)


class ReplicaBroadcast:
    """``broadcast(obj_or_None)`` with the calling convention of ``dist.broadcast_object_list``:
    the leader passes the object, the others pass ``None`` and get the leader's object back."""

    def __init__(self, is_leader: bool, num_followers: int, address: Optional[Dict[str, Any]] = None):
        self.is_leader = is_leader
        self.server = ZmqServer(num_followers) if is_leader else None
        self.client = None if is_leader else ZmqClient(address)

    @property
    def address(self):
        return self.server.address if self.server is not None else None

    def broadcast(self, obj: Any = None) -> Any:
        if self.is_leader:
            self.server.broadcast(obj)
            return obj
        return self.client.receive()


def setup_replica_broadcast(group, src_global_rank: int, group_size: int, is_leader: bool) -> Optional[ReplicaBroadcast]:
    """Build the side channel for one replica: the leader starts a server and its address is
    shared over ``group`` once; afterwards no collective is needed for small host messages."""
    import torch.distributed as dist

    if group_size <= 1 or not dist.is_initialized():
        return None
    leader = ReplicaBroadcast(True, group_size - 1) if is_leader else None
    box = [leader.address if is_leader else None]
    dist.broadcast_object_list(box, src=src_global_rank, group=group)
    if is_leader:
        leader.server.wait_for_clients()
        return leader
    return ReplicaBroadcast(False, 0, box[0])
