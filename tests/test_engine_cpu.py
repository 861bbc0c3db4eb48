"""Rollout engine: decode steps launched one ahead of the host give exactly the tokens of the
step-by-step loop (sampling, n samples per prompt, end-of-sequence stops, length stops, more
requests than sequence slots)."""
import torch

from mindspeed_rl_b200.models.gpt import GPTModel
from mindspeed_rl_b200.models.transformer_config import TransformerConfig
from mindspeed_rl_b200.reshard.alias import alias_rollout_weights
from mindspeed_rl_b200.rollout.engine import LLMEngine
from mindspeed_rl_b200.rollout.scheduler import SamplingParams


def _engine(lookahead: bool):
    torch.manual_seed(5)
    cfg = TransformerConfig(num_layers=2, hidden_size=32, ffn_hidden_size=64, num_attention_heads=4,
                            num_query_groups=2, vocab_size=48, params_dtype=torch.float32,
                            max_position_embeddings=128)
    m = GPTModel(cfg, device="cpu")
    for p in m.parameters():
        p.data.mul_(3.0)
    eng = LLMEngine(cfg, "cpu", max_num_seqs=6, max_num_batched_tokens=64, max_model_len=40, block_size=4,
                    eos_token_id=7, seed=11)
    eng.lookahead_decode = lookahead
    eng.runner.bind_weights(alias_rollout_weights(m))
    eng.init_cache(64)
    return eng


def _run(lookahead: bool):
    eng = _engine(lookahead)
    prompts = [[3, 9, 27, 5], [1, 2, 3, 4, 5, 6], [11, 12], [20, 21, 22]]
    params = SamplingParams(n=3, temperature=1.0, max_tokens=12, seed=3)
    outs = eng.generate(prompts, params)
    return [(o.request_id is not None, [(c.token_ids, c.finish_reason, [round(x, 5) for x in c.logprobs])
                                        for c in o.outputs]) for o in outs], eng.stats["steps"]


def test_lookahead_decode_is_exact():
    a, steps_a = _run(False)
    b, steps_b = _run(True)
    assert a == b
    reasons = {c[1] for _, outs in a for c in outs}
    assert reasons == {"length", "stop"}             # the case covers both ways a sequence ends
    assert steps_a == steps_b


def test_abort_returns_partial_output_and_frees_blocks():
    """A request that is aborted between steps hands back what it has produced so far, its cache blocks return
    to the pool, and the remaining requests finish as if it had never been queued beside them."""
    eng = _engine(lookahead=False)
    free0 = eng.bm.num_free_blocks
    params = SamplingParams(n=1, temperature=0.0, max_tokens=10)
    eng.add_request("keep", [3, 9, 27, 5], params)
    eng.add_request("drop", [1, 2, 3, 4, 5, 6], params)
    for _ in range(4):
        eng.step()
    assert eng.get_num_unfinished_requests() == 2 and eng.bm.num_free_blocks < free0
    out = eng.abort_request("drop")
    assert out is not None and out.request_id == "drop" and 1 <= len(out.outputs[0].token_ids) < 10
    assert eng.abort_request("drop") is None and eng.abort_request("never-queued") is None
    assert eng.get_num_unfinished_requests() == 1
    done = []
    while eng.has_unfinished_requests():
        done += [o for o in eng.step() if o.finished]
    assert [o.request_id for o in done] == ["keep"]
    assert eng.bm.num_free_blocks == free0                      # every block came back
    alone = _engine(lookahead=False)
    ref = alone.generate([[3, 9, 27, 5]], params)[0]
    assert done[0].outputs[0].token_ids == ref.outputs[0].token_ids
    assert eng.kv_bytes_per_block() == 2 * 2 * 4 * 2 * 8 * 4     # K and V x layers x block x kv heads x head dim x fp32


def test_prompt_at_the_length_limit_finishes_without_tokens():
    """A prompt that already fills ``max_model_len`` is answered at once with finish reason "length" and no
    tokens; the requests queued behind it are served normally."""
    eng = _engine(lookahead=False)
    params = SamplingParams(n=1, temperature=0.0, max_tokens=4)
    outs = eng.generate([list(range(1, 41)), [3, 9, 27, 5]], params)       # max_model_len is 40
    assert outs[0].outputs[0].token_ids == [] and outs[0].outputs[0].finish_reason == "length"
    assert len(outs[1].outputs[0].token_ids) >= 1 and outs[1].finished
    assert not eng.has_unfinished_requests()
