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
