"""Chat templates with tools and thinking, dataset handlers and padding helpers, rendered through a character
tokenizer so that the produced text can be read back."""
import json
import os
from types import SimpleNamespace

import pytest
import torch

from mindspeed_rl_b200.datasets import templates as T

TEMPLATES = os.path.join(os.path.dirname(__file__), "..", "configs", "model", "templates.json")
SPECIAL = 0x110000


class CharTok:
    """Characters map to their code points, registered special strings to ids above the Unicode range."""

    def __init__(self):
        self.specials = ["<|endoftext|>"]
        self.eos_token = None
        self.pad_token = None
        self.bos_token_id = None
        self.vocab_size = SPECIAL + 64

    def _id(self, tok):
        if tok not in self.specials:
            self.specials.append(tok)
        return SPECIAL + self.specials.index(tok)

    @property
    def eos_token_id(self):
        return None if self.eos_token is None else self._id(self.eos_token)

    @property
    def pad_token_id(self):
        return None if self.pad_token is None else self._id(self.pad_token)

    def convert_tokens_to_ids(self, tok):
        return self._id(tok)

    def add_special_tokens(self, d, replace_additional_special_tokens=True):
        for name in ("eos_token", "pad_token"):                  # as the Hugging Face classes do: set and register
            if name in d:
                setattr(self, name, d[name])
                self._id(d[name])
        for t in d.get("additional_special_tokens", []):
            self._id(t)

    def encode(self, text, add_special_tokens=False, **_):
        return [ord(c) for c in text]

    def text(self, ids):
        return "".join(self.specials[i - SPECIAL] if i >= SPECIAL else chr(i) for i in ids)


WEATHER = {"name": "get_weather", "description": "Weather of a city",
           "parameters": {"type": "object", "required": ["city"],
                          "properties": {"city": {"type": "string", "description": "City name"},
                                         "unit": {"type": "string", "enum": ["C", "F"], "description": "Unit"},
                                         "days": {"type": "array", "items": {"type": "integer"}, "description": "Days"}}}}


def test_tool_and_function_formatters():
    text = T.default_tool_formatter([WEATHER])
    assert "> Tool Name: get_weather" in text and "- city (string, required): City name" in text
    assert "should be one of [C, F]" in text and "where each item should be integer" in text
    assert "Action: tool name (one of [get_weather])" in text
    q = T.qwen_tool_formatter([WEATHER])
    assert "<tools>" in q and json.dumps({"type": "function", "function": WEATHER}) in q and "<tool_call>" in q
    assert T.default_tool_extractor('Action: get_weather\nAction Input: {"city": "Paris"}') == \
        ("get_weather", '{"city": "Paris"}')
    assert T.default_tool_extractor("just talking") == "just talking"
    assert T.default_tool_extractor("Action: f\nAction Input: {broken") == "Action: f\nAction Input: {broken"
    tools = T.ToolFormatter(tool_format="default")
    assert tools.apply(content=json.dumps([WEATHER])) == [text] and tools.apply(content="[]") == [""]
    assert tools.apply(content="not json") == [""] and tools.extract("just talking") == "just talking"
    assert T.ToolFormatter(tool_format="qwen").apply(content=json.dumps([WEATHER])) == [q]
    call = json.dumps({"name": "get_weather", "arguments": {"city": "Paris"}})
    fn = T.FunctionFormatter(slots=["Action: {{name}}\nAction Input: {{arguments}}"], tool_format="default")
    assert fn.apply(content=call) == ['Action: get_weather\nAction Input: {"city": "Paris"}']
    assert fn.apply(content="garbage") == ["Action: \nAction Input: "]
    qfn = T.FunctionFormatter(slots=["{{content}}<|im_end|>\n"], tool_format="qwen")
    assert qfn.apply(content=call) == ['<tool_call>\n{"name": "get_weather", "arguments": {"city": "Paris"}}\n</tool_call><|im_end|>\n']
    with pytest.raises(ValueError):
        T.EmptyFormatter(slots=["{{content}}"])
    with pytest.raises(ValueError):
        T.StringFormatter(slots=["no placeholder"])
    with pytest.raises(TypeError):
        T.StringFormatter(slots=["{{content}}"]).apply(content=3)


def test_qwen3_template_with_tools_and_thinking():
    tok = CharTok()
    tpl = T.fix_model_tokenizer(tok, "qwen3", TEMPLATES)
    assert tok.eos_token == "<|im_end|>" and tok.pad_token == "<|im_end|>"       # stop word replaces EOS, pad follows
    msgs = [{"role": "user", "content": "weather in Paris?"},
            {"role": "assistant", "content": "<think>call the tool</think>\n\nchecking"},
            {"role": "user", "content": "and tomorrow?"},
            {"role": "assistant", "content": "sunny"}]
    pairs = tpl.encode_multiturn(tok, msgs, "be brief", json.dumps([WEATHER]))
    assert len(pairs) == 2
    first = tok.text(pairs[0][0])
    assert "be brief" in first and "<tools>" in first and "weather in Paris?" in first
    assert "call the tool" not in tok.text(pairs[0][1])               # earlier thoughts are stripped from history
    assert tok.text(pairs[0][1]).startswith("checking")
    last = tok.text(pairs[1][1])
    assert last.startswith("<think>\n\n</think>\n\nsunny")            # thinking off: an empty thought is pre-filled
    thinking = T.get_model_template("qwen3", TEMPLATES, enable_thinking=True)
    assert tok.text(thinking.encode_multiturn(tok, msgs)[1][1]).startswith("sunny")
    # a trailing user turn (an RL prompt) comes back as a query without answer
    prompt, answer = tpl.encode_oneturn(tok, msgs[:3], None, None)
    assert answer == [] and tok.text(prompt).rstrip().endswith("<|im_start|>assistant")
    # observation and function turns
    tool_msgs = [{"role": "user", "content": "q"},
                 {"role": "function", "content": json.dumps({"name": "get_weather", "arguments": {"city": "Paris"}})},
                 {"role": "observation", "content": "18C"}, {"role": "assistant", "content": "18 degrees"}]
    rendered = "".join(tok.text(a) + tok.text(b) for a, b in tpl.encode_multiturn(tok, tool_msgs))
    assert '<tool_call>\n{"name": "get_weather"' in rendered and "18C" in rendered
    with pytest.raises(NotImplementedError):
        tpl.encode_multiturn(tok, [{"role": "narrator", "content": "x"}])
    with pytest.raises(ValueError):
        T.get_model_template("no_such_template", TEMPLATES)


def test_cutoff_shares_length_between_prompt_and_answer():
    assert T.infer_max_len(30, 10, 20, 1) == (15, 5)
    assert T.infer_max_len(100, 1, 10, 4) == (9, 1) and T.infer_max_len(0, 0, 10, 1) == (0, 0)
    tok = CharTok()
    tpl = T.get_model_template("empty", TEMPLATES)
    pairs = tpl.encode_multiturn(tok, [{"role": "user", "content": "a" * 30}, {"role": "assistant", "content": "b" * 10}],
                                 cutoff_len=20)
    assert len(pairs[0][0]) + len(pairs[0][1]) <= 20 and len(pairs[0][1]) >= 1


def _handler_args(tmp_path, **kw):
    base = dict(prompt_type="qwen", prompt_type_path=TEMPLATES, dataset_additional_keys=[], output_prefix=str(tmp_path / "d"),
                map_keys=None, log_interval=1000, append_eod=False, enable_thinking=False, placeholder_token="@",
                reward_tokens=["+", "-"])
    base.update(kw)
    return SimpleNamespace(**base)


def test_instruction_and_process_reward_handlers(tmp_path):
    from mindspeed_rl_b200.datasets.data_handler import (AlpacaStyleInstructionHandler,
                                                         AlpacaStyleProcessRewardHandler)
    tok = CharTok()
    tok.eos_token = "<|im_end|>"
    rows = [{"instruction": "add 1 and 2", "input": "", "output": "3"}]
    h = AlpacaStyleInstructionHandler(_handler_args(tmp_path), rows, tok)
    (sample,) = list(h.get_tokenized_data())
    ids, labels = sample["input_ids"], sample["labels"]
    assert len(ids) == len(labels) == len(sample["attention_mask"])
    text = tok.text(ids)
    assert "<|im_start|>user\nadd 1 and 2<|im_end|>" in text and "<|im_start|>assistant\n3" in text
    n_ans = sum(1 for l in labels if l != -100)
    assert 0 < n_ans < len(ids) and tok.text([l for l in labels if l != -100]).startswith("3")
    assert all(l == -100 or l == i for l, i in zip(labels, ids))      # labels are the ids wherever they count
    # process reward data: every step marker is labelled with its verdict token, the rest ignored
    prm_rows = [{"instruction": "s1 @ s2 @", "input": "", "output": '["+", "-"]'},
                {"instruction": "s1 @ s2 @", "input": "", "output": '["+"]'}]             # marker count mismatch: dropped
    prm = AlpacaStyleProcessRewardHandler(_handler_args(tmp_path, prompt_type="empty"), prm_rows, tok)
    out = list(prm.get_tokenized_data())
    assert len(out) == 1
    marks = [(i, l) for i, l in enumerate(out[0]["labels"]) if l != -100]
    assert [tok.text([out[0]["input_ids"][i]]) for i, _ in marks] == ["@", "@"]
    assert [chr(l) for _, l in marks] == ["+", "-"]


def test_padding_helpers():
    from mindspeed_rl_b200.utils.pad_process import (remove_padding_and_split_to_list, response_window,
                                                     truncate_middle_and_pad, truncate_prompt_and_pad)
    resp = torch.tensor([[5, 6, 2, 0, 0], [7, 8, 9, 10, 11], [2, 0, 0, 0, 0]])
    rows = remove_padding_and_split_to_list(resp, eos_token_id=2, pad_token_id=0)
    assert [r.tolist() for r in rows] == [[5, 6, 2], [7, 8, 9, 10, 11], [2]]
    rows = remove_padding_and_split_to_list(torch.tensor([[5, 6, 2, 2, 2], [7, 8, 9, 10, 11]]), 2, 2)
    assert [r.tolist() for r in rows] == [[5, 6, 2], [7, 8, 9, 10, 11]]                 # pad == eos: the first one is kept
    assert remove_padding_and_split_to_list(torch.tensor([[5, 6, 2, 2, 2]]), 2, 2, to_list=True) == [[5, 6]]
    win = response_window(torch.tensor([[3], [1]]), torch.tensor([[2], [4]]))
    assert win.tolist() == [[2, 4], [0, 4]]
    x = torch.arange(12).reshape(2, 6)
    assert truncate_prompt_and_pad(torch.zeros(2, 4), x, win, pad_value=-1).tolist() == [[2, 3, -1, -1], [6, 7, 8, 9]]
    x3 = x.unsqueeze(-1).float().expand(2, 6, 2)
    got = truncate_middle_and_pad(torch.zeros(2, 4), x3, win, pad_value=0.0)
    assert got.shape == (2, 4, 2) and got[0, :, 0].tolist() == [2.0, 3.0, 0.0, 0.0]


def test_hugging_face_tokenizer_wrapper_with_a_local_vocabulary(tmp_path):
    """A word-level tokenizer saved in the Hugging Face layout, loaded through the wrapper with a chat template:
    the template's stop word becomes EOS, pad falls back to EOS, and the rule reward decodes with it."""
    from types import SimpleNamespace as NS
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast
    from mindspeed_rl_b200.rewards.registry import compute_verifier_score
    from mindspeed_rl_b200.utils.tokenizer import get_tokenizer

    vocab = {"<unk>": 0, "<eos>": 1}
    for w in "user assistant add and the answer is \\boxed{3} \\boxed{4} 1 2 3 4 <|im_start|>".split(" "):
        vocab.setdefault(w, len(vocab))
    raw = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    raw.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    PreTrainedTokenizerFast(tokenizer_object=raw, unk_token="<unk>", eos_token="<eos>").save_pretrained(str(tmp_path))
    tok = get_tokenizer(str(tmp_path), "HuggingFaceTokenizer", "qwen", TEMPLATES)
    assert tok.tokenizer.eos_token == "<|im_end|>" and tok.eod == tok.pad == len(vocab)     # added as a special token
    assert tok.vocab_size == len(vocab) + 1 and tok.vocab["add"] == vocab["add"]
    ids = tok.tokenize("add 1 and 2")
    assert ids == [vocab[w] for w in ("add", "1", "and", "2")] and tok.detokenize(ids) == "add 1 and 2"
    assert tok.template is not None and tok.template.stop_words == ["<|im_end|>"]
    # rule reward over token rows: -100 in the labels is mapped to EOS and dropped with the special tokens
    resp = [torch.tensor(tok.tokenize("the answer is \\boxed{3}") + [tok.eod]),
            torch.tensor(tok.tokenize("the answer is \\boxed{4}"))]
    labels = [torch.tensor(tok.tokenize("3") + [-100]), torch.tensor(tok.tokenize("3"))]
    cfg = NS(verifier_function=["math_17k_acc"], verifier_weight=[2.0], verifier_parallel=1)
    scores, metrics, _ = compute_verifier_score({"responses": resp, "labels": labels,
                                                 "response_length": [torch.tensor([6]), torch.tensor([5])]}, cfg, tok)
    assert scores.tolist() == [2.0, 0.0] and metrics["math_17k_acc_rewards/mean"] == [1.0, 0.0]
