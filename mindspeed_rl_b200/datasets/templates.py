"""Chat templates: render multi-turn conversations into token ids.

A template is a set of slot *formatters* (user / assistant / system / function / observation /
tools / separator / prefix) plus flags, loaded by name from ``configs/model/templates.json``.
``Template.encode_oneturn`` returns ``(prompt ids, answer ids)`` where the prompt holds every
earlier turn and the last query; ``encode_multiturn`` returns one pair per turn.  Rendering:
turn 0 = ``prefix + system(+tools) + user``, later user turns = ``separator + user``.
Slots are strings with ``{{content}}`` / ``{{idx}}`` placeholders, ``{"token": "<...>"}`` dicts for
literal special tokens and ``["bos_token"]`` / ``["eos_token"]`` lists for tokenizer specials.

Reference behaviour: ``mindspeed_rl/datasets/templates.py:41-469``, ``datasets/formatter.py:29-188``.
"""
from __future__ import annotations

import json
import re
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple, Union

Slot = Union[str, Dict[str, str], List[str]]

_PLACEHOLDER = re.compile(r"\{\{([a-zA-Z_][a-zA-Z0-9_]*)\}\}")

TOOL_SYSTEM_PROMPT = (
    "You have access to the following tools:\n{tool_text}"
    "Use the following format if using a tool:\n```\n"
    "Action: tool name (one of [{tool_names}]).\n"
    "Action Input: the input to the tool, as a JSON object of the form "
    "```{{\"input\": \"hello world\", \"num_beams\": 5}}```.\n```\n")


def default_tool_formatter(tools: List[Dict[str, Any]]) -> str:
    text, names = "", []
    for tool in tools:
        params = ""
        props = tool.get("parameters", {}).get("properties", {})
        required = tool.get("parameters", {}).get("required", [])
        for name, p in props.items():
            extras = (", required" if name in required else "")
            if p.get("enum"):
                extras += ", should be one of [{}]".format(", ".join(p["enum"]))
            if p.get("items"):
                extras += ", where each item should be {}".format(p["items"].get("type", ""))
            params += "  - {} ({}{}): {}\n".format(name, p.get("type", ""), extras, p.get("description", ""))
        text += "> Tool Name: {}\nTool Description: {}\nTool Args:\n{}\n".format(
            tool["name"], tool.get("description", ""), params)
        names.append(tool["name"])
    return TOOL_SYSTEM_PROMPT.format(tool_text=text, tool_names=", ".join(names))


def qwen_tool_formatter(tools: List[Dict[str, Any]]) -> str:
    body = "\n".join(json.dumps({"type": "function", "function": t}, ensure_ascii=False) for t in tools)
    return ("\n\n# Tools\n\nYou may call one or more functions to assist with the user query.\n\n"
            "You are provided with function signatures within <tools></tools> XML tags:\n<tools>\n"
            f"{body}\n</tools>\n\nFor each function call, return a json object with function name and "
            "arguments within <tool_call></tool_call> XML tags:\n<tool_call>\n"
            "{\"name\": <function-name>, \"arguments\": <args-json-object>}\n</tool_call>")


def default_tool_extractor(content: str) -> Union[str, Tuple[str, str]]:
    m = re.search(r"Action:\s*([a-zA-Z0-9_]+).*?Action Input:\s*(.*)", content, re.DOTALL)
    if not m:
        return content
    raw = m.group(2).strip().strip('"').strip("`")
    try:
        return m.group(1).strip(), json.dumps(json.loads(raw), ensure_ascii=False)
    except json.JSONDecodeError:
        return content


@dataclass
class Formatter:
    slots: List[Slot] = field(default_factory=list)
    tool_format: Optional[str] = None

    def apply(self, **kwargs) -> List[Slot]:
        raise NotImplementedError

    def extract(self, content: str):
        raise NotImplementedError


@dataclass
class EmptyFormatter(Formatter):
    def __post_init__(self):
        if any(isinstance(s, str) and _PLACEHOLDER.search(s) for s in self.slots):
            raise ValueError("an empty formatter must not contain placeholders")

    def apply(self, **kwargs):
        return self.slots


@dataclass
class StringFormatter(Formatter):
    def __post_init__(self):
        if not any(isinstance(s, str) and _PLACEHOLDER.search(s) for s in self.slots):
            raise ValueError("a string formatter needs at least one placeholder")

    def apply(self, **kwargs):
        out: List[Slot] = []
        for slot in self.slots:
            if isinstance(slot, str):
                for k, v in kwargs.items():
                    if not isinstance(v, str):
                        raise TypeError(f"placeholder '{k}' expects a string")
                    slot = slot.replace("{{" + k + "}}", v, 1)
                out.append(slot)
            elif isinstance(slot, (dict, list, set)):
                out.append(slot)
            else:
                raise TypeError(f"unsupported slot {slot!r}")
        return out


@dataclass
class FunctionFormatter(StringFormatter):
    """Assistant tool call: content is ``{"name": ..., "arguments": {...}}`` JSON."""

    def __post_init__(self):
        pass

    def apply(self, **kwargs):
        content = kwargs.pop("content")
        try:
            call = json.loads(content)
            name, args = call["name"], json.dumps(call["arguments"], ensure_ascii=False)
        except Exception:
            name, args = "", ""
        if self.tool_format == "qwen":
            text = f"<tool_call>\n{{\"name\": \"{name}\", \"arguments\": {args}}}\n</tool_call>"
            return StringFormatter.apply(self, content=text)
        out = []
        for slot in self.slots:
            out.append(slot.replace("{{name}}", name).replace("{{arguments}}", args).replace(
                "{{content}}", f"Action: {name}\nAction Input: {args}") if isinstance(slot, str) else slot)
        return out


@dataclass
class ToolFormatter(Formatter):
    def apply(self, **kwargs):
        content = kwargs.pop("content")
        try:
            tools = json.loads(content)
            if not tools:
                return [""]
            fmt = qwen_tool_formatter if self.tool_format == "qwen" else default_tool_formatter
            return [fmt(tools)]
        except Exception:
            return [""]

    def extract(self, content: str):
        return default_tool_extractor(content)


@dataclass
class Template:
    format_user: Formatter
    format_assistant: Formatter
    format_system: Formatter
    format_function: Formatter
    format_observation: Formatter
    format_tools: Formatter
    format_separator: Formatter
    format_prefix: Formatter
    default_system: str = ""
    stop_words: List[str] = field(default_factory=list)
    efficient_eos: bool = False
    replace_eos: bool = False
    force_system: bool = False
    enable_thinking: bool = False
    thought_words: Tuple[str, str] = ("<think>", "</think>")

    def encode_oneturn(self, tokenizer, messages: List[Dict[str, str]], system: Optional[str] = None,
                       tools: Optional[str] = None, cutoff_len: int = 1_000_000,
                       reserved_label_len: int = 1) -> Tuple[List[int], List[int]]:
        pairs = self._encode(tokenizer, messages, system, tools, cutoff_len, reserved_label_len)
        prompt: List[int] = []
        for q, r in pairs[:-1]:
            prompt += q + r
        return prompt + pairs[-1][0], pairs[-1][1]

    def encode_multiturn(self, tokenizer, messages, system=None, tools=None, cutoff_len: int = 1_000_000,
                         reserved_label_len: int = 1) -> List[Tuple[List[int], List[int]]]:
        return self._encode(tokenizer, messages, system, tools, cutoff_len, reserved_label_len)

    def _encode(self, tokenizer, messages, system, tools, cutoff_len, reserved_label_len):
        system = system or self.default_system
        encoded = []
        for i, msg in enumerate(messages):
            elems: List[Slot] = []
            if i == 0:
                elems += self.format_prefix.apply()
                if system or tools:
                    tool_text = self.format_tools.apply(content=tools)[0] if tools else ""
                    elems += self.format_system.apply(content=system + tool_text)
            elif i % 2 == 0:
                elems += self.format_separator.apply()
            role, content = msg["role"], msg["content"]
            if role == "user":
                elems += self.format_user.apply(content=content, idx=str(i // 2))
            elif role == "assistant":
                elems += self.format_assistant.apply(content=content)
            elif role == "observation":
                elems += self.format_observation.apply(content=content)
            elif role == "function":
                elems += self.format_function.apply(content=content)
            else:
                raise NotImplementedError(f"unexpected role '{role}'")
            encoded.append(self._to_ids(tokenizer, elems))
        return self._make_pairs(encoded, cutoff_len, reserved_label_len)

    @staticmethod
    def _to_ids(tokenizer, elems: Sequence[Slot]) -> List[int]:
        ids: List[int] = []
        for e in elems:
            if isinstance(e, str):
                if e:
                    ids += tokenizer.encode(e, add_special_tokens=False)
            elif isinstance(e, dict):
                ids += [tokenizer.convert_tokens_to_ids(e.get("token"))]
            elif isinstance(e, (list, set)):
                if "bos_token" in e and tokenizer.bos_token_id is not None:
                    ids.append(tokenizer.bos_token_id)
                elif "eos_token" in e and tokenizer.eos_token_id is not None:
                    ids.append(tokenizer.eos_token_id)
            else:
                raise TypeError(f"unsupported element {e!r}")
        return ids

    @staticmethod
    def _make_pairs(encoded: List[List[int]], cutoff_len: int, reserved_label_len: int):
        pairs, total = [], 0
        for i in range(0, len(encoded) - 1, 2) if len(encoded) > 1 else []:
            if total >= cutoff_len:
                break
            src, tgt = encoded[i], encoded[i + 1]
            s_len, t_len = infer_max_len(len(src), len(tgt), cutoff_len - total, reserved_label_len)
            pairs.append((src[:s_len], tgt[:t_len]))
            total += s_len + t_len
        if len(encoded) % 2 == 1:  # trailing query without answer (RL prompts)
            pairs.append((encoded[-1][:max(cutoff_len - total, 0)], []))
        return pairs


class ReasoningTemplate(Template):
    """Template for thinking models: strips earlier ``<think>...</think>`` from history and, with
    thinking disabled, pre-fills an empty thought in the answer."""

    def _encode(self, tokenizer, messages, system, tools, cutoff_len, reserved_label_len):
        msgs = [dict(m) for m in messages]
        lo, hi = self.thought_words
        pat = re.compile(re.escape(lo) + r".*?" + re.escape(hi) + r"\s*", re.DOTALL)
        for m in msgs[:-1]:
            if m["role"] == "assistant":
                m["content"] = pat.sub("", m["content"])
        if msgs and msgs[-1]["role"] == "assistant" and not self.enable_thinking \
                and lo not in msgs[-1]["content"]:
            msgs[-1]["content"] = f"{lo}\n\n{hi}\n\n" + msgs[-1]["content"]
        return super()._encode(tokenizer, msgs, system, tools, cutoff_len, reserved_label_len)


def infer_max_len(source_len: int, target_len: int, max_len: int, reserved_label_len: int) -> Tuple[int, int]:
    """Share ``max_len`` between source and target proportionally, keeping room for the label."""
    if source_len + target_len == 0:
        return 0, 0
    max_target = max(int(max_len * (target_len / (source_len + target_len))), reserved_label_len)
    max_source = max_len - min(max_target, target_len)
    return min(source_len, max_source), min(target_len, max_target)


def _formatter(spec: Optional[Dict[str, Any]], default: Formatter, kind: str) -> Formatter:
    if spec is None:
        return default
    slots = spec.get("slots", [])
    tool_format = spec.get("tool_format")
    if kind == "tools":
        return ToolFormatter(slots=slots, tool_format=tool_format or "default")
    if kind == "function":
        return FunctionFormatter(slots=slots or ["{{content}}"], tool_format=tool_format)
    has_ph = any(isinstance(s, str) and _PLACEHOLDER.search(s) for s in slots)
    return StringFormatter(slots=slots, tool_format=tool_format) if has_ph else \
        EmptyFormatter(slots=slots, tool_format=tool_format)


_templates: Dict[str, Template] = {}


def register_template(spec: Dict[str, Any], enable_thinking: bool = False) -> Template:
    eos = [] if not spec.get("efficient_eos") else [["eos_token"]]
    d_user = StringFormatter(slots=["{{content}}"])
    d_assistant = StringFormatter(slots=["{{content}}"] + eos)
    cls = ReasoningTemplate if spec.get("template_class") == "ReasoningTemplate" else Template
    tpl = cls(
        format_user=_formatter(spec.get("format_user"), d_user, "user"),
        format_assistant=_formatter(spec.get("format_assistant"), d_assistant, "assistant"),
        format_system=_formatter(spec.get("format_system"), d_user, "system"),
        format_function=_formatter(spec.get("format_function"),
                                   FunctionFormatter(slots=["Action: {{name}}\nAction Input: {{arguments}}"] + eos),
                                   "function"),
        format_observation=_formatter(spec.get("format_observation"),
                                      _formatter(spec.get("format_user"), d_user, "user"), "observation"),
        format_tools=_formatter(spec.get("format_tools"), ToolFormatter(tool_format="default"), "tools"),
        format_separator=_formatter(spec.get("format_separator"), EmptyFormatter(), "separator"),
        format_prefix=_formatter(spec.get("format_prefix"), EmptyFormatter(), "prefix"),
        default_system=spec.get("default_system", ""), stop_words=list(spec.get("stop_words", [])),
        efficient_eos=bool(spec.get("efficient_eos", False)), replace_eos=bool(spec.get("replace_eos", False)),
        force_system=bool(spec.get("force_system", False)), enable_thinking=enable_thinking)
    _templates[spec["name"]] = tpl
    return tpl


def get_model_template(name: str, prompt_type_path: str, enable_thinking: bool = False) -> Template:
    """Load the template ``name`` from a ``templates.json`` file."""
    with open(prompt_type_path, "r", encoding="utf-8") as fh:
        specs = json.load(fh)
    for spec in specs:
        if spec["name"] == name:
            return register_template(spec, enable_thinking)
    raise ValueError(f"prompt type '{name}' not found in {prompt_type_path} "
                     f"(available: {[s['name'] for s in specs]})")


def fix_model_tokenizer(tokenizer, name: str, prompt_type_path: str, enable_thinking: bool = False) -> Template:
    """Apply a template's special-token requirements (stop words become EOS / extra specials)."""
    tpl = get_model_template(name, prompt_type_path, enable_thinking)
    stops = list(tpl.stop_words)
    def set_eos(token: str) -> None:
        # registering it as a special token also adds it to the vocabulary when the model file lacks it
        try:
            tokenizer.add_special_tokens({"eos_token": token})
        except Exception:
            tokenizer.eos_token = token

    if tpl.replace_eos and stops:
        set_eos(stops.pop(0))
    if tokenizer.eos_token_id is None:
        set_eos("<|endoftext|>")
    if tokenizer.pad_token_id is None:
        tokenizer.pad_token = tokenizer.eos_token
    if stops:
        tokenizer.add_special_tokens({"additional_special_tokens": stops}, replace_additional_special_tokens=False)
    return tpl
