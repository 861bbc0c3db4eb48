"""Tools and the multi-turn rollout loop (CPU)."""
import json

import torch

from mindspeed_rl_b200.tools.base import (BaseTool, FunctionSchema, HermesToolParser, ToolParser, build_tool_map,
                                          register_tool)
from mindspeed_rl_b200.tools.builtin import ExecutionPool, ReTool, SandboxFusionTool, SearchTool, TokenBucket
from mindspeed_rl_b200.tools.multi_turn import (MultiTurnRollout, TurnState, process_response, truncate_tool_text)


class CharTokenizer:
    """One token per character (ids = code points), enough for the parser and the loop."""

    def encode(self, text, add_special_tokens=False):
        return [min(ord(c), 1023) for c in text]

    def decode(self, ids):
        return "".join(chr(i) for i in ids)


@register_tool("EchoTool")
class EchoTool(BaseTool):
    def execute(self, instance_id, parameters, **kw):
        if parameters.get("boom"):
            raise RuntimeError("tool failure")
        return "echo:" + json.dumps(parameters, sort_keys=True), 0.0, {}


def test_hermes_parser_and_truncation():
    p = ToolParser.get_tool_parser("hermes", CharTokenizer())
    assert isinstance(p, HermesToolParser)
    text = 'a<tool_call>{"name": "f", "arguments": {"x": 1}}</tool_call>b<tool_call>{bad json}</tool_call>' \
           '<tool_call>{"name": "g", "arguments": {}}</tool_call>'
    calls = p.extract_tool_calls(CharTokenizer().encode(text))
    assert [(c.name, c.argument_dict()) for c in calls] == [("f", {"x": 1}), ("g", {})]
    assert p.extract_from_text("no calls here") == []
    s = "0123456789" * 3
    assert truncate_tool_text(s, 10, "left") == s[:10] + "...(truncated)"
    assert truncate_tool_text(s, 10, "right") == "(truncated)..." + s[-10:]
    assert truncate_tool_text(s, 10, "middle") == s[:5] + "...(truncated)..." + s[-5:]
    assert truncate_tool_text("short", 10) == "short"


def test_sandbox_retool_search_with_fake_transport():
    seen = []

    def transport(url, payload, timeout):
        seen.append((url, payload))
        if "queries" in payload:
            return {"result": [[{"document": {"contents": "Title A\nbody a"}}, {"document": {"contents": "T2\nb2"}}]]}
        return {"status": "Success", "run_result": {"status": "Finished", "stdout": "4\n", "stderr": ""}}

    sb = SandboxFusionTool({"sandbox_fusion_url": "http://x/run", "transport": transport})
    iid = sb.create()
    assert sb.execute(iid, {"code": "print(2+2)"})[0] == "4\n"
    sb.release(iid)
    rt = ReTool({"sandbox_fusion_url": "http://x/run", "transport": transport})
    rt.execute(rt.create(), {"code": "```python\nx = 2\nx + 2\n```"})
    assert seen[-1][1]["code"] == "x = 2\nprint(x + 2)"
    failing = SandboxFusionTool({"sandbox_fusion_url": "u", "transport": lambda *a: {"status": "Failed"}})
    assert failing.execute(failing.create(), {"code": "1"})[0] == "no stdout here"
    st = SearchTool({"retrieval_service_url": "http://x/retrieve", "transport": transport, "topk": 2})
    text, _, meta = st.execute(st.create(), {"query_list": ["q"]})
    assert "Doc 1 (Title: Title A)" in json.loads(text)["result"] and meta["total_results"] == 2
    assert "missing" in st.execute(st.create(), {})[0]


def test_execution_pool_rate_limit():
    import threading
    import time

    pool = ExecutionPool(num_workers=8, enable_global_rate_limit=False, rate_limit=2)
    peak, live, lock = [0], [0], threading.Lock()

    def job():
        with lock:
            live[0] += 1
            peak[0] = max(peak[0], live[0])
        time.sleep(0.02)
        with lock:
            live[0] -= 1
        return 1

    assert sum(f.result() for f in [pool.submit(job) for _ in range(8)]) == 8
    assert peak[0] <= 2
    assert TokenBucket(3).rate_limit == 3


def test_process_response_rules():
    tok = CharTokenizer()
    tools = build_tool_map([{"class_name": "EchoTool", "tool_schema": FunctionSchema("echo").to_openai()}])
    parser = ToolParser.get_tool_parser("hermes", tok)
    cfg = dict(max_total_response_length=400, max_tool_calls=2, max_parallel_calls=1, max_tool_response_length=8)
    call = tok.encode('<tool_call>{"name": "echo", "arguments": {"q": "abcdefghijklmnop"}}</tool_call>')
    ids = process_response(tools, parser, tok, TurnState(call, [1] * len(call), 0), cfg)
    text = tok.decode(ids)
    assert text.startswith("<|im_start|>user\n<tool_response>\necho...(truncated)...op\"}\n</tool_response>")
    assert text.endswith("<|im_end|>\n<|im_start|>assistant\n")
    assert process_response(tools, parser, tok, TurnState(call, [1] * len(call), 2), cfg) == []      # tool budget
    assert process_response(tools, parser, tok, TurnState(call, [1] * 400, 0), cfg) == []           # length budget
    assert process_response(tools, parser, tok, TurnState(tok.encode("plain"), [1] * 5, 0), cfg) == []
    boom = tok.encode('<tool_call>{"name": "echo", "arguments": {"boom": true}}</tool_call>')
    assert process_response(tools, parser, tok, TurnState(boom, [1] * len(boom), 0), cfg) == []
    tight = dict(cfg, max_total_response_length=len(call) + 10)
    assert process_response(tools, parser, tok, TurnState(call, [1] * len(call), 0), tight) == []   # would overflow


def test_multi_turn_loop_on_real_engine():
    """Tiny random model on CPU: the first turn of every sample is followed by a scripted tool
    turn; the same request id is re-queued with the whole context (prefix cache hit)."""
    from mindspeed_rl_b200.models.gpt import GPTModel
    from mindspeed_rl_b200.models.transformer_config import TransformerConfig
    from mindspeed_rl_b200.reshard.alias import alias_rollout_weights
    from mindspeed_rl_b200.rollout.engine import LLMEngine
    from mindspeed_rl_b200.rollout.scheduler import SamplingParams

    cfg = TransformerConfig(num_layers=2, hidden_size=64, ffn_hidden_size=128, num_attention_heads=4,
                            num_query_groups=2, vocab_size=1024, params_dtype=torch.float32)
    model = GPTModel(cfg, device="cpu", seed=0)
    eng = LLMEngine(cfg, "cpu", max_num_seqs=8, max_num_batched_tokens=512, max_model_len=256, block_size=8,
                    enable_prefix_caching=True, eos_token_id=-1)
    eng.runner.bind_weights(alias_rollout_weights(model))
    eng.init_cache(256)
    tok = CharTokenizer()
    tools = build_tool_map([{"class_name": "EchoTool", "tool_schema": FunctionSchema("echo").to_openai()}])
    mt = MultiTurnRollout(eng, tok, tools, "hermes", vocab_size=1024, max_total_response_length=120,
                          max_tool_calls=1, max_parallel_calls=1, max_tool_response_length=16)

    class Scripted(HermesToolParser):
        def extract_tool_calls(self, ids):
            return self.extract_from_text('<tool_call>{"name": "echo", "arguments": {"k": 1}}</tool_call>')

    mt.parser = Scripted(tok)
    prompts = [[5, 6, 7, 8, 9, 10, 11, 12, 13], [20, 21, 22, 23]]
    res = mt.generate(prompts, SamplingParams(max_tokens=16, temperature=1.0, seed=0))
    assert len(res) == 2
    for p, r in zip(prompts, res):
        assert r["prompt_ids"] == p and r["tool_call_num"] == 1
        assert r["input_ids"] == p + r["responses"] and len(r["response_mask"]) == r["response_length"] <= 120
        zeros = [i for i, m in enumerate(r["response_mask"]) if m == 0]
        assert zeros and zeros == list(range(zeros[0], zeros[-1] + 1))        # one contiguous tool turn
        tool_text = tok.decode([r["responses"][i] for i in zeros])
        assert tool_text.startswith("<|im_start|>user\n<tool_response>") and zeros[0] == 16
        assert r["response_mask"][-1] == 1                                   # a second model turn followed
    assert eng.bm.stats()["prefix_hits"] > 0 if hasattr(eng.bm, "stats") else True
