"""Host runtime pieces: ZeroMQ replica broadcast (ordering, re-send after a dropped message,
time-out when a follower never acknowledges)."""
import threading

import pytest

from mindspeed_rl_b200.runtime.zmq_broadcast import ZmqClient, ZmqServer


def _follow(address, n_msgs, out, cls=ZmqClient):
    c = cls(address)
    out.append([c.receive(timeout=20) for _ in range(n_msgs)])
    c.close()


def test_broadcast_in_order_to_all_followers():
    server = ZmqServer(num_clients=3, resend_interval=0.2)
    got = []
    threads = [threading.Thread(target=_follow, args=(server.address, 5, got)) for _ in range(3)]
    for t in threads:
        t.start()
    server.wait_for_clients(timeout=20)
    msgs = [{"step": i, "payload": list(range(i))} for i in range(5)]
    for m in msgs:
        server.broadcast(m)
    for t in threads:
        t.join(20)
    assert len(got) == 3 and all(g == msgs for g in got)
    server.close()


class _LossyClient(ZmqClient):
    """Loses the first copy of message 2 (neither delivers nor acknowledges it)."""
    dropped = False

    def receive(self, timeout=120.0):
        import pickle
        import time
        deadline = time.time() + timeout
        while time.time() < deadline:
            if not self.sub.poll(200):
                continue
            seq_b, payload = self.sub.recv_multipart()
            seq = int(seq_b)
            if seq == 2 and not self.dropped:
                self.dropped = True            # the message is lost on the wire
                continue
            self.push.send_multipart([self.id.encode(), seq_b])
            if seq == self.next_seq:
                self.next_seq += 1
                return pickle.loads(payload)
        raise TimeoutError


def test_dropped_message_is_resent():
    server = ZmqServer(num_clients=1, resend_interval=0.1)
    got = []
    t = threading.Thread(target=_follow, args=(server.address, 3, got, _LossyClient))
    t.start()
    server.wait_for_clients(timeout=20)
    for i in range(3):
        server.broadcast(i)
    t.join(20)
    assert got == [[0, 1, 2]]
    server.close()


def test_missing_acknowledgement_times_out():
    server = ZmqServer(num_clients=1, resend_interval=0.02, max_resends=3)
    server.clients.add("ghost")                # registered but never answers
    with pytest.raises(TimeoutError):
        server.broadcast("hello")
    server.close()


def test_change_gate_chooses_the_tier_from_the_changed_files():
    import importlib.util
    import os
    spec = importlib.util.spec_from_file_location(
        "access_control_test", os.path.join(os.path.dirname(__file__), "..", "ci", "access_control_test.py"))
    gate = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gate)
    assert gate.choose_tier(["README.md", "profiles/x.md", "examples/grpo/a.sh"]) == "skip"
    assert gate.choose_tier(["tests/test_units_cpu.py", "NOTES.md"]) == "cpu"
    assert gate.choose_tier(["tests/test_gpu_kernels.py"]) == "build"
    assert gate.choose_tier(["mindspeed_rl_b200/csrc/decode.cu"]) == "build"
    assert gate.choose_tier([]) == "build"
    assert gate.commands_for("skip", gpu=True) == []
    assert len(gate.commands_for("cpu", gpu=True)) == 1
    cmds = gate.commands_for("build", gpu=True)
    assert len(cmds) == 3 and cmds[-1][-1] == "gpu" and "build()" in cmds[0][-1]
    assert len(gate.commands_for("build", gpu=False)) == 2
    assert gate.main(["--files-from", os.devnull, "--dry-run"]) == 0


def test_rpc_errors_timeouts_and_concurrent_callers():
    """Remote calls: an exception on the serving side arrives as RemoteError with its traceback text, a server
    that does not answer in time gives TimeoutError (and the proxy is usable again afterwards), and calls from
    several threads are served side by side."""
    import threading
    import time
    import pytest
    from mindspeed_rl_b200.runtime.rpc import ActorProxy, RemoteError, serve

    class Target:
        def __init__(self):
            self.live, self.peak, self.lock = 0, 0, threading.Lock()

        def add(self, a, b=0):
            return a + b

        def boom(self):
            raise KeyError("no such row")

        def slow(self, seconds):
            with self.lock:
                self.live += 1
                self.peak = max(self.peak, self.live)
            time.sleep(seconds)
            with self.lock:
                self.live -= 1
            return seconds

    target = Target()
    server = serve(target, num_threads=4)
    try:
        proxy = ActorProxy(server.address, timeout_s=2.0)
        assert proxy._call("__ping__") == "pong" and proxy.add(2, b=3) == 5
        with pytest.raises(RemoteError) as err:
            proxy.boom()
        assert "KeyError" in str(err.value) and "no such row" in str(err.value) and "boom" in str(err.value)
        with pytest.raises(RemoteError):
            proxy.no_such_method()
        assert proxy.add(1, 1) == 2                                   # the connection survives remote errors
        results = []
        threads = [threading.Thread(target=lambda: results.append(proxy.slow(0.2))) for _ in range(4)]
        t0 = time.time()
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        assert results == [0.2] * 4 and target.peak >= 2 and time.time() - t0 < 0.75
        quick = ActorProxy(server.address, timeout_s=0.1)
        with pytest.raises(TimeoutError):
            quick.slow(0.5)
        time.sleep(0.5)
        assert quick.add(4, 4) == 8                                   # a fresh socket after the timeout
        with pytest.raises(AttributeError):
            proxy._private
    finally:
        server.shutdown()
    gone = ActorProxy(server.address, timeout_s=0.3)
    time.sleep(0.3)
    with pytest.raises(TimeoutError):
        gone.add(1, 2)
