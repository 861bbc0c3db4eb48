"""Built-in tools: remote code sandbox (plain and "ReTool" flavour) and retrieval search, plus
the bounded execution pool they share.

Behavioural parity (reference: ``mindspeed_rl/tools/sandbox_fusion_tool.py:14-71``,
``tools/retool.py:12-40``, ``tools/search_tool.py:16-89``, ``tools/utils/execution_pool.py:12-60``):

* calls go through a worker pool of ``num_workers`` threads gated by a token bucket of
  ``rate_limit`` concurrent requests (process-wide when ``enable_global_rate_limit``);
* the sandbox posts ``{code, language, run_timeout, memory_limit_MB}`` to ``sandbox_fusion_url`` and
  returns ``stdout + stderr`` of a finished run, otherwise the literal ``"no stdout here"``;
* ReTool first pulls the code out of a ```` ```python ```` fence and wraps a trailing bare
  expression in ``print(...)``;
* search posts ``{queries, topk, return_scores}`` to ``retrieval_service_url`` and renders the hits
  as ``Doc i (Title: ...)`` passages inside ``{"result": ...}``.

The HTTP transport is injectable (``config["transport"]``: ``callable(url, payload, timeout) ->
dict``) so the tools can be exercised without a network.
"""
from __future__ import annotations

import json
import re
import threading
from concurrent.futures import ThreadPoolExecutor
from typing import Any, Callable, Dict, List, Optional, Tuple

from .base import BaseTool, FunctionSchema, register_tool


class TokenBucket:
    """At most ``rate_limit`` holders at a time."""

    def __init__(self, rate_limit: int):
        self.rate_limit = int(rate_limit)
        self._sem = threading.Semaphore(self.rate_limit)
        self._lock = threading.Lock()
        self.current = 0

    def acquire(self) -> None:
        self._sem.acquire()
        with self._lock:
            self.current += 1

    def release(self) -> None:
        with self._lock:
            self.current -= 1
        self._sem.release()


_GLOBAL_BUCKETS: Dict[int, TokenBucket] = {}
_GLOBAL_LOCK = threading.Lock()


class ExecutionPool:
    def __init__(self, num_workers: int = 10, enable_global_rate_limit: bool = True, rate_limit: int = 10):
        self._pool = ThreadPoolExecutor(max_workers=max(int(num_workers), 1))
        if enable_global_rate_limit:
            with _GLOBAL_LOCK:
                self._bucket = _GLOBAL_BUCKETS.setdefault(int(rate_limit), TokenBucket(rate_limit))
        else:
            self._bucket = TokenBucket(rate_limit)

    def submit(self, fn: Callable, *args, **kwargs):
        def run():
            self._bucket.acquire()
            try:
                return fn(*args, **kwargs)
            finally:
                self._bucket.release()
        return self._pool.submit(run)

    def execute(self, fn: Callable, *args, **kwargs):
        return self.submit(fn, *args, **kwargs).result()


def http_post_json(url: str, payload: Dict[str, Any], timeout: float) -> Dict[str, Any]:
    import requests

    resp = requests.post(url, json=payload, timeout=timeout, headers={"Content-Type": "application/json"})
    resp.raise_for_status()
    return resp.json()


class _RemoteTool(BaseTool):
    def __init__(self, config, schema, default_workers: int, default_rate: int):
        super().__init__(config, schema)
        c = self.config
        self.pool = ExecutionPool(c.get("num_workers", default_workers), c.get("enable_global_rate_limit", True),
                                  c.get("rate_limit", default_rate))
        self.transport: Callable = c.get("transport") or http_post_json

    def create(self, instance_id: Optional[str] = None, ground_truth: Optional[str] = None, **kwargs) -> str:
        iid = super().create(instance_id)
        self._instances[iid] = {"response": "", "ground_truth": ground_truth, "reward": []}
        return iid

    def calc_reward(self, instance_id: str, **kwargs):
        return self._instances[instance_id]["reward"]


@register_tool("SandboxFusionTool")
class SandboxFusionTool(_RemoteTool):
    def __init__(self, config: Optional[Dict[str, Any]] = None, schema: Optional[FunctionSchema] = None):
        super().__init__(config, schema or FunctionSchema(
            "code_interpreter", "Run a piece of code and return what it prints.",
            {"type": "object", "properties": {"code": {"type": "string"}}, "required": ["code"]}), 10, 10)
        c = self.config
        self.url = c.get("sandbox_fusion_url", "")
        if not self.url:
            raise ValueError("sandbox_fusion_url is not set")
        self.default_timeout = c.get("default_timeout", 30)
        self.default_language = c.get("default_language", "python")
        self.memory_limit_mb = c.get("memory_limit_mb", 1024)

    def prepare_code(self, code: str) -> str:
        return code

    def run_code(self, code: str, timeout: float, language: str) -> str:
        payload = {"code": code, "language": language, "run_timeout": timeout, "compile_timeout": timeout,
                   "memory_limit_MB": self.memory_limit_mb}
        try:
            reply = self.transport(self.url, payload, timeout + 10)
        except Exception:
            return "no stdout here"
        run = (reply or {}).get("run_result") or {}
        if (reply or {}).get("status") == "Success" and run.get("status") == "Finished":
            return (run.get("stdout") or "") + (run.get("stderr") or "")
        return "no stdout here"

    def execute(self, instance_id: str, parameters: Dict[str, Any], **kwargs) -> Tuple[str, float, Dict[str, Any]]:
        code = parameters.get("code", "")
        code = self.prepare_code(code if isinstance(code, str) else str(code))
        out = self.pool.execute(self.run_code, code, parameters.get("timeout", self.default_timeout),
                                parameters.get("language", self.default_language))
        return out, 0.0, {}


@register_tool("ReTool")
class ReTool(SandboxFusionTool):
    _fence = re.compile(r"```python(.*?)```", re.DOTALL)

    def prepare_code(self, code: str) -> str:
        m = self._fence.findall(code)
        if m:
            code = m[0].strip()
        lines = code.split("\n")
        for i in range(len(lines) - 1, -1, -1):
            if lines[i] == "":
                continue
            if not lines[i].startswith("print"):
                lines[i] = f"print({lines[i]})"
            break
        return "\n".join(lines)


def passages_to_string(hits: List[Dict[str, Any]]) -> str:
    out = []
    for i, hit in enumerate(hits):
        doc = hit.get("document", hit)
        content = (doc.get("contents") or "").strip()
        title, _, text = content.partition("\n")
        out.append(f"Doc {i + 1} (Title: {title})\n{text}\n")
    return "\n".join(out).strip()


@register_tool("SearchTool")
class SearchTool(_RemoteTool):
    def __init__(self, config: Optional[Dict[str, Any]] = None, schema: Optional[FunctionSchema] = None):
        super().__init__(config, schema or FunctionSchema(
            "search", "Search a corpus for passages relevant to the queries.",
            {"type": "object", "properties": {"query_list": {"type": "array", "items": {"type": "string"}}},
             "required": ["query_list"]}), 120, 120)
        c = self.config
        self.url = c.get("retrieval_service_url")
        if self.url == "":
            raise ValueError("retrieval_service_url is not set")
        self.timeout = c.get("timeout", 30)
        self.topk = c.get("topk", 3)

    def run_search(self, queries: List[str]) -> Tuple[str, Dict[str, Any]]:
        meta = {"query_count": len(queries), "status": "unknown", "total_results": 0, "api_request_error": None}
        try:
            reply = self.transport(self.url, {"queries": queries, "topk": self.topk, "return_scores": True},
                                   self.timeout)
        except Exception as e:
            meta.update(status="api_error", api_request_error=str(e))
            return json.dumps({"result": f"Search request failed: {e}"}), meta
        results = (reply or {}).get("result") or []
        texts = [passages_to_string(hits) for hits in results]
        meta.update(status="success" if texts else "no_results", total_results=sum(len(h) for h in results))
        if not texts:
            return json.dumps({"result": "No search results found."}), meta
        return json.dumps({"result": "\n---\n".join(texts)}, ensure_ascii=False), meta

    def execute(self, instance_id: str, parameters: Dict[str, Any], **kwargs) -> Tuple[str, float, Dict[str, Any]]:
        queries = parameters.get("query_list")
        if not queries or not isinstance(queries, list):
            return json.dumps({"result": "Error: 'query_list' is missing, empty, or not a list in parameters."}), 0.0, {}
        try:
            text, meta = self.pool.execute(self.run_search, queries)
        except Exception as e:
            return json.dumps({"result": f"Search execution failed: {e}"}), 0.0, {"error": str(e)}
        self._instances.setdefault(instance_id, {"reward": []})["reward"].append(text.strip())
        return text, 0.0, meta
