"""Multi-turn tool-use rollouts on top of the rollout engine's request API.

``process_response`` decides what follows a finished generation turn (reference:
``mindspeed_rl/tools/utils/tool_utils.py:75-135``): nothing when the response budget or the tool
budget is used up, when no ``<tool_call>`` parses, when a tool raises, or when the tool turn would
overflow the budget; otherwise up to ``max_parallel_calls`` tools run (create -> execute ->
release), every result is cut to ``max_tool_response_length`` characters (left / right / middle)
and the results are wrapped as a user turn holding ``<tool_response>`` blocks followed by the
assistant header, tokenised without special tokens.

``MultiTurnRollout.generate`` drives the loop (reference:
``mindspeed_rl/workers/actor_hybrid_worker.py:667-796``): every prompt is a request; when a turn
finishes, out-of-vocabulary ids are zeroed, its tokens get mask 1, the tool turn's tokens mask 0,
and the *whole* context is re-submitted under the same request id -- the engine's prefix cache
makes the re-submission cost only the new tokens.  The response of a sample is everything after
the original prompt, truncated to ``max_total_response_length``.
"""
from __future__ import annotations

import uuid
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence

from .base import BaseTool, ParsedToolCall, ToolParser

USER_OPEN = "<|im_start|>user\n"
TURN_CLOSE_ASSISTANT_OPEN = "<|im_end|>\n<|im_start|>assistant\n"


def truncate_tool_text(text: str, max_len: int, side: str = "middle") -> str:
    if not text or len(text) <= max_len:
        return text
    if side == "left":
        return text[:max_len] + "...(truncated)"
    if side == "right":
        return "(truncated)..." + text[-max_len:]
    half = max_len // 2
    return text[:half] + "...(truncated)..." + text[-half:]


def call_tool(tool_map: Dict[str, BaseTool], call: ParsedToolCall, tools_kwargs: Dict[str, Any]) -> str:
    tool = tool_map[call.name]
    kw = (tools_kwargs or {}).get(call.name, {})
    iid = tool.create(**kw.get("create_kwargs", {}))
    try:
        text, _, _ = tool.execute(iid, call.argument_dict(), **kw.get("execute_kwargs", {}))
    finally:
        tool.release(iid)
    return text


@dataclass
class TurnState:
    """What ``process_response`` needs to know about one sample."""
    response_ids: List[int]
    response_mask: List[int]
    tool_call_num: int = 0


def process_response(tool_map: Dict[str, BaseTool], parser: ToolParser, tokenizer, state: TurnState,
                     cfg: Dict[str, Any], tools_kwargs: Optional[Dict[str, Any]] = None) -> List[int]:
    """Token ids of the tool turn to append, or ``[]`` when the conversation ends here."""
    max_total = cfg["max_total_response_length"]
    if len(state.response_mask) >= max_total or state.tool_call_num >= cfg.get("max_tool_calls", 1):
        return []
    calls = parser.extract_tool_calls(state.response_ids)
    if not calls:
        return []
    calls = calls[:cfg.get("max_parallel_calls", 1)]
    try:
        results = [call_tool(tool_map, c, tools_kwargs or {}) for c in calls]
    except Exception:
        return []
    limit = cfg.get("max_tool_response_length", 256)
    side = cfg.get("tool_response_truncate_side", "middle")
    body = "".join(f"<tool_response>\n{truncate_tool_text(str(r), limit, side)}\n</tool_response>" for r in results)
    text = USER_OPEN + body + TURN_CLOSE_ASSISTANT_OPEN
    ids = list(tokenizer.encode(text, add_special_tokens=False))
    if len(state.response_mask) + len(ids) >= max_total:
        return []
    return ids


@dataclass
class MultiTurnSample:
    prompt_ids: List[int]
    context: List[int] = field(default_factory=list)
    response_mask: List[int] = field(default_factory=list)
    tool_call_num: int = 0
    done: bool = False


class MultiTurnRollout:
    def __init__(self, engine, tokenizer, tool_map: Dict[str, BaseTool], parser_name: str = "hermes", *,
                 vocab_size: int, max_total_response_length: int, max_tool_calls: int = 1,
                 max_parallel_calls: int = 1, max_tool_response_length: int = 256,
                 tool_response_truncate_side: str = "middle", tools_kwargs: Optional[Dict[str, Any]] = None,
                 share_result: Optional[Callable[[List[int]], List[int]]] = None):
        """``share_result``: hook that makes a tool turn identical on all ranks of a rollout TP
        group (rank 0 computes, the others receive); identity when ``None``."""
        self.engine, self.tokenizer, self.tool_map = engine, tokenizer, tool_map
        self.parser = ToolParser.get_tool_parser(parser_name, tokenizer)
        self.vocab_size = vocab_size
        self.cfg = dict(max_total_response_length=max_total_response_length, max_tool_calls=max_tool_calls,
                        max_parallel_calls=max_parallel_calls, max_tool_response_length=max_tool_response_length,
                        tool_response_truncate_side=tool_response_truncate_side)
        self.tools_kwargs = tools_kwargs or {}
        self.share_result = share_result or (lambda ids: ids)

    def _params(self, base, used: int, ctx_len: int):
        import dataclasses

        # a turn is bounded by the context window, the remaining response budget and the
        # per-turn ``max_tokens`` of the sampling config
        room = min(self.engine.max_model_len - ctx_len, self.cfg["max_total_response_length"] - used,
                   base.max_tokens or (1 << 30))
        return dataclasses.replace(base, n=1, max_tokens=max(int(room), 1))

    def generate(self, prompts: Sequence[Sequence[int]], sampling_params) -> List[Dict[str, Any]]:
        samples: Dict[str, MultiTurnSample] = {}
        tag = uuid.uuid4().hex[:6]
        for i, p in enumerate(prompts):
            rid = f"req_{i}_{tag}"
            s = MultiTurnSample(list(p), list(p))
            samples[rid] = s
            self.engine.add_request(rid, s.context, self._params(sampling_params, 0, len(s.context)))
        while self.engine.any_unfinished_requests():
            for out in self.engine.step():
                if not out.finished:
                    continue
                s = samples[out.request_id]
                new = [t if t < self.vocab_size else 0 for t in out.outputs[0].token_ids]
                s.context += new
                s.response_mask += [1] * len(new)
                state = TurnState(new, s.response_mask, s.tool_call_num)
                tool_ids = self.share_result(
                    process_response(self.tool_map, self.parser, self.tokenizer, state, self.cfg, self.tools_kwargs))
                room = self.engine.max_model_len - len(s.context) - len(tool_ids)
                if not tool_ids or room <= 0:
                    s.done = True
                    continue
                s.context += tool_ids
                s.response_mask += [0] * len(tool_ids)
                s.tool_call_num += 1
                self.engine.add_request(out.request_id, s.context,
                                        self._params(sampling_params, len(s.response_mask), len(s.context)))
        results = []
        limit = self.cfg["max_total_response_length"]
        for rid in sorted(samples, key=lambda r: int(r.split("_")[1])):
            s = samples[rid]
            resp = s.context[len(s.prompt_ids):][:limit]
            results.append(dict(prompt_ids=s.prompt_ids, responses=resp, response_mask=s.response_mask[:limit],
                                input_ids=s.prompt_ids + resp, response_length=len(resp),
                                tool_call_num=s.tool_call_num))
        return results
