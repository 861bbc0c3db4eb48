"""Worker processes for grading calls that must not outlive a wall-clock limit.

A grading call may hand a model-written string to sympy, which can run for minutes.  A thread
cannot be stopped, so a call that has to be *ended* runs in a child process: every worker serves
one call at a time over a pipe; a call that passes its limit gets the default result, its worker is
killed and a fresh one takes its place.  The pool is persistent (starting an interpreter costs far
more than a grading call) and is shared by all verifiers of a process.

Reference behaviour: the global process pool of the rule verifiers with a 1 s limit per call
(``mindspeed_rl/models/rule_verifier.py:23-77,197-205``) and the subprocess-with-queue
``call_with_timeout`` of the grader (``mindspeed_rl/utils/math_eval_toolkit/grader.py``).
"""
from __future__ import annotations

import atexit
import multiprocessing as mp
import time
from multiprocessing.connection import wait
from typing import Any, Callable, List, Optional, Sequence


def _import(name: str) -> bool:
    """Import ``name`` in the worker and run its ``warm_up()`` when it has one (slow first-use set-up that
    must not count against a call's limit)."""
    import sys

    __import__(name)
    init = getattr(sys.modules[name], "warm_up", None)
    if callable(init):
        init()
    return True


def _serve(conn) -> None:
    """Child: answer ``(fn, args)`` with ``(True, result)`` or ``(False, repr(error))`` until EOF."""
    while True:
        try:
            job = conn.recv()
        except (EOFError, OSError):
            return
        if job is None:
            return
        fn, args = job
        try:
            conn.send((True, fn(*args)))
        except Exception as e:          # the caller maps a failed call to its default
            try:
                conn.send((False, repr(e)))
            except Exception:
                return


class _Worker:
    def __init__(self, ctx):
        self.conn, child = ctx.Pipe()
        self.proc = ctx.Process(target=_serve, args=(child,), daemon=True)
        self.proc.start()
        child.close()
        self.job: Optional[int] = None       # index of the item in flight
        self.deadline = 0.0
        self.warm = set()                    # modules this worker has imported

    def stop(self, kill: bool = False) -> None:
        try:
            if kill:
                self.proc.kill()
            else:
                self.conn.send(None)
        except Exception:
            pass
        try:
            self.conn.close()
        except Exception:
            pass
        self.proc.join(timeout=1.0)
        if self.proc.is_alive():
            self.proc.kill()
            self.proc.join(timeout=1.0)


class BoundedPool:
    """``map(fn, items, timeout)``: ``fn(*item)`` for every item, each under its own limit.

    ``fn`` and the items must be picklable (module-level functions, plain data).  Results come back
    in item order; an item that timed out, raised, or lost its worker yields ``default``.
    """

    def __init__(self, workers: int = 4, start_method: Optional[str] = None):
        methods = mp.get_all_start_methods()
        method = start_method or ("forkserver" if "forkserver" in methods else "spawn")
        self.ctx = mp.get_context(method)
        self.size = max(1, int(workers))
        self.workers: List[_Worker] = []
        self.timeouts = 0            # calls ended by their limit since the pool was built
        self.restarts = 0            # workers replaced

    def _grow(self, n: int) -> None:
        while len(self.workers) < min(self.size, n):
            self.workers.append(_Worker(self.ctx))

    def _replace(self, w: _Worker) -> _Worker:
        w.stop(kill=True)
        self.restarts += 1
        fresh = _Worker(self.ctx)
        self.workers[self.workers.index(w)] = fresh
        return fresh

    def _warm_up(self, module: str, limit: float = 120.0) -> None:
        """Import ``module`` in every worker that has not seen it, all at once: the first import of a large
        package takes seconds, which must not count against the first call's limit."""
        cold = [w for w in self.workers if module not in w.warm]
        for w in cold:
            try:
                w.conn.send((_import, (module,)))
            except Exception:
                pass
        end = time.monotonic() + limit
        for w in cold:
            try:
                if w.conn.poll(max(0.0, end - time.monotonic())):
                    w.conn.recv()
                    w.warm.add(module)
                    continue
            except (EOFError, OSError):
                pass
            self._replace(w)

    def map(self, fn: Callable, items: Sequence[Sequence[Any]], timeout: float = 1.0, default: Any = None,
            total_timeout: Optional[float] = None) -> List[Any]:
        """``total_timeout`` bounds the whole batch: items not finished by then yield ``default``."""
        n = len(items)
        out: List[Any] = [default] * n
        if n == 0:
            return out
        self._grow(n)
        self._warm_up(getattr(fn, "__module__", None) or "builtins")
        end = None if total_timeout is None else time.monotonic() + total_timeout
        nxt = 0
        busy = 0

        def give(w: _Worker) -> None:
            nonlocal nxt, busy
            while nxt < n:
                i = nxt
                nxt += 1
                try:
                    w.conn.send((fn, tuple(items[i])))
                except Exception:            # unpicklable item or dead worker: default for this item
                    if not w.proc.is_alive():
                        w = self._replace(w)
                    continue
                w.job, w.deadline = i, time.monotonic() + timeout
                busy += 1
                return
            w.job = None

        for w in list(self.workers):
            give(w)
        while busy:
            now = time.monotonic()
            if end is not None and now >= end:
                for w in list(self.workers):
                    if w.job is not None:
                        self._replace(w)
                        self.timeouts += 1
                return out
            running = [w for w in self.workers if w.job is not None]
            limit = min(w.deadline for w in running)
            if end is not None:
                limit = min(limit, end)
            ready = wait([w.conn for w in running], timeout=max(0.0, limit - now))
            now = time.monotonic()
            for w in running:
                if w.conn in ready:
                    try:
                        ok, val = w.conn.recv()
                        if ok:
                            out[w.job] = val
                    except (EOFError, OSError):           # the worker died under the call
                        w = self._replace(w)
                    busy -= 1
                    give(w)
                elif now >= w.deadline:
                    self.timeouts += 1
                    busy -= 1
                    give(self._replace(w))
        return out

    def close(self) -> None:
        for w in self.workers:
            w.stop()
        self.workers = []


_pool: Optional[BoundedPool] = None
_parallel = 1


def set_parallel(n: int) -> None:
    """Number of grading processes used by ``bounded_map`` (1: grade in the calling process)."""
    global _parallel, _pool
    n = max(1, int(n))
    if _pool is not None and _pool.size != n:
        _pool.close()
        _pool = None
    _parallel = n


def parallel() -> int:
    return _parallel


def shared_pool() -> BoundedPool:
    global _pool
    if _pool is None:
        _pool = BoundedPool(_parallel)
    return _pool


@atexit.register
def _shutdown() -> None:
    global _pool
    if _pool is not None:
        _pool.close()
        _pool = None
