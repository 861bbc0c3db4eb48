"""Minimal actor RPC over ZeroMQ: serve any Python object's methods to other processes.

``serve(obj, bind)`` starts a ROUTER front-end and a pool of worker threads (so that slow
calls such as a blocking ``get_experience`` do not stall the others -- the experience store
is designed for concurrent access).  ``connect(address)`` returns a proxy whose attribute
calls are forwarded; tensors travel through pickle protocol 5.  This is the transport of
the built-in runtime when Ray is not installed (the reference uses Ray actors with
``max_concurrency=100``: ``mindspeed_rl/trainer/utils/transfer_dock.py:248``).
"""
from __future__ import annotations

import pickle
import threading
import traceback
import uuid
from typing import Any, Optional

import zmq


class RemoteError(RuntimeError):
    pass


class ActorServer:
    def __init__(self, obj: Any, bind: str = "tcp://127.0.0.1:0", num_threads: int = 8):
        self.obj = obj
        self.ctx = zmq.Context.instance()
        self.front = self.ctx.socket(zmq.ROUTER)
        if bind.endswith(":0"):
            port = self.front.bind_to_random_port(bind[:-2])
            self.address = f"{bind[:-2]}:{port}"
        else:
            self.front.bind(bind)
            self.address = bind
        self._inproc = f"inproc://actor-{uuid.uuid4().hex}"
        self.back = self.ctx.socket(zmq.DEALER)
        self.back.bind(self._inproc)
        self._stop = threading.Event()
        self._threads = [threading.Thread(target=self._worker, daemon=True) for _ in range(num_threads)]
        self._proxy = threading.Thread(target=self._run_proxy, daemon=True)
        for t in self._threads:
            t.start()
        self._proxy.start()

    def _run_proxy(self) -> None:
        poller = zmq.Poller()
        poller.register(self.front, zmq.POLLIN)
        poller.register(self.back, zmq.POLLIN)
        while not self._stop.is_set():
            try:
                events = dict(poller.poll(100))
            except zmq.ZMQError:
                break
            if self.front in events:
                self.back.send_multipart(self.front.recv_multipart())
            if self.back in events:
                self.front.send_multipart(self.back.recv_multipart())
        self.front.close(0)
        self.back.close(0)

    def _worker(self) -> None:
        sock = self.ctx.socket(zmq.REP)
        sock.connect(self._inproc)
        sock.setsockopt(zmq.RCVTIMEO, 200)
        while not self._stop.is_set():
            try:
                msg = sock.recv()
            except zmq.Again:
                continue
            except zmq.ZMQError:
                break
            try:
                method, args, kwargs = pickle.loads(msg)
                if method == "__ping__":
                    result = "pong"
                else:
                    result = getattr(self.obj, method)(*args, **kwargs)
                payload = pickle.dumps(("ok", result), protocol=5)
            except Exception as e:  # noqa: BLE001 - forwarded to the caller
                payload = pickle.dumps(("err", f"{type(e).__name__}: {e}\n{traceback.format_exc()}"),
                                       protocol=5)
            sock.send(payload)
        sock.close(0)

    def shutdown(self) -> None:
        self._stop.set()


class ActorProxy:
    """Client side: ``proxy.method(*args)`` performs a blocking remote call.  One socket per
    calling thread."""

    def __init__(self, address: str, timeout_s: Optional[float] = None):
        self._address = address
        self._timeout = timeout_s
        self._local = threading.local()

    def _sock(self):
        s = getattr(self._local, "sock", None)
        if s is None:
            s = zmq.Context.instance().socket(zmq.REQ)
            s.setsockopt(zmq.LINGER, 0)
            if self._timeout:
                s.setsockopt(zmq.RCVTIMEO, int(self._timeout * 1000))
            s.connect(self._address)
            self._local.sock = s
        return s

    def _call(self, method: str, *args, **kwargs):
        s = self._sock()
        s.send(pickle.dumps((method, args, kwargs), protocol=5))
        try:
            status, value = pickle.loads(s.recv())
        except zmq.Again:
            s.close(0)
            self._local.sock = None
            raise TimeoutError(f"remote call {method} to {self._address} timed out")
        if status == "err":
            raise RemoteError(value)
        return value

    def __getattr__(self, name: str):
        if name.startswith("_"):
            raise AttributeError(name)
        return lambda *a, **kw: self._call(name, *a, **kw)


def serve(obj: Any, bind: str = "tcp://127.0.0.1:0", num_threads: int = 8) -> ActorServer:
    return ActorServer(obj, bind, num_threads)


def connect(address: str, timeout_s: Optional[float] = None) -> ActorProxy:
    return ActorProxy(address, timeout_s)
