"""Tool abstractions for multi-turn rollouts: schemas, the tool base class, the registry and the
Hermes ``<tool_call>`` parser.

A tool follows a ``create -> execute -> release`` life cycle per call (reference:
``mindspeed_rl/tools/base_tool.py:12-37``); tools are looked up by the ``name`` of their
OpenAI-style function schema (``tools/utils/schemas.py:25-81``, ``tool_registry.py:7-41``).
The parser decodes a response and returns every well-formed
``<tool_call>{"name": ..., "arguments": {...}}</tool_call>`` block
(``tools/utils/tool_parser.py:56-80``); malformed JSON blocks are skipped.
"""
from __future__ import annotations

import importlib
import json
import re
import uuid
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple, Type


@dataclass
class FunctionSchema:
    name: str
    description: str = ""
    parameters: Dict[str, Any] = field(default_factory=lambda: {"type": "object", "properties": {}, "required": []})

    def to_openai(self) -> Dict[str, Any]:
        return {"type": "function", "function": {"name": self.name, "description": self.description,
                                                 "parameters": self.parameters}}

    @classmethod
    def from_openai(cls, d: Dict[str, Any]) -> "FunctionSchema":
        f = d.get("function", d)
        return cls(f["name"], f.get("description", ""), f.get("parameters", {"type": "object", "properties": {}}))


@dataclass
class ParsedToolCall:
    name: str
    arguments: str          # JSON text of the argument object

    def argument_dict(self) -> Dict[str, Any]:
        out = json.loads(self.arguments)
        if not isinstance(out, dict):
            raise ValueError("tool arguments must be a JSON object")
        return out


class BaseTool:
    """Sub-classes override ``execute`` (and ``create`` / ``release`` when they hold state)."""

    def __init__(self, config: Optional[Dict[str, Any]] = None, schema: Optional[FunctionSchema] = None):
        self.config = dict(config or {})
        self.schema = schema or FunctionSchema(type(self).__name__)
        self.name = self.schema.name
        self._instances: Dict[str, Dict[str, Any]] = {}

    def get_openai_tool_schema(self) -> Dict[str, Any]:
        return self.schema.to_openai()

    def create(self, instance_id: Optional[str] = None, **kwargs) -> str:
        iid = instance_id or uuid.uuid4().hex
        self._instances[iid] = dict(kwargs)
        return iid

    def execute(self, instance_id: str, parameters: Dict[str, Any], **kwargs) -> Tuple[str, float, Dict[str, Any]]:
        """Returns ``(response text, step reward, metrics)``."""
        raise NotImplementedError

    def calc_reward(self, instance_id: str, **kwargs) -> float:
        return 0.0

    def release(self, instance_id: str, **kwargs) -> None:
        self._instances.pop(instance_id, None)


_TOOL_CLASSES: Dict[str, Type[BaseTool]] = {}


def register_tool(name: str):
    def deco(cls: Type[BaseTool]) -> Type[BaseTool]:
        _TOOL_CLASSES[name] = cls
        return cls
    return deco


def resolve_tool_class(path: str) -> Type[BaseTool]:
    """``registered name`` or dotted ``module.ClassName``."""
    if path in _TOOL_CLASSES:
        return _TOOL_CLASSES[path]
    module, _, cls = path.rpartition(".")
    if not module:
        raise KeyError(f"unknown tool '{path}'")
    return getattr(importlib.import_module(module), cls)


def build_tool_map(tool_configs: List[Dict[str, Any]]) -> Dict[str, BaseTool]:
    """``[{class_name, config, tool_schema}]`` (the layout of a tools YAML) -> ``{name: tool}``."""
    out: Dict[str, BaseTool] = {}
    for entry in tool_configs or []:
        cls = resolve_tool_class(entry["class_name"])
        schema = FunctionSchema.from_openai(entry["tool_schema"]) if entry.get("tool_schema") else None
        tool = cls(entry.get("config"), schema)
        out[tool.name] = tool
    return out


def load_tool_map(yaml_path: str) -> Dict[str, BaseTool]:
    import yaml

    with open(yaml_path) as fh:
        return build_tool_map((yaml.safe_load(fh) or {}).get("tools", []))


# ---- parsers -------------------------------------------------------------------------------------------
class ToolParser:
    _registry: Dict[str, Type["ToolParser"]] = {}

    def __init__(self, tokenizer):
        self.tokenizer = tokenizer

    def extract_tool_calls(self, response_ids: List[int]) -> List[ParsedToolCall]:
        raise NotImplementedError

    @classmethod
    def register(cls, name: str):
        def deco(sub):
            cls._registry[name] = sub
            return sub
        return deco

    @classmethod
    def get_tool_parser(cls, name: str, tokenizer) -> "ToolParser":
        if name not in cls._registry:
            raise ValueError(f"unknown tool parser '{name}'")
        return cls._registry[name](tokenizer)


@ToolParser.register("hermes")
class HermesToolParser(ToolParser):
    START, END = "<tool_call>", "</tool_call>"
    _block = re.compile(r"<tool_call>(.*?)</tool_call>", re.DOTALL)

    def extract_from_text(self, text: str) -> List[ParsedToolCall]:
        if self.START not in text or self.END not in text:
            return []
        calls = []
        for body in self._block.findall(text):
            try:
                obj = json.loads(body)
                calls.append(ParsedToolCall(obj["name"], json.dumps(obj["arguments"], ensure_ascii=False)))
            except (ValueError, KeyError, TypeError):
                continue
        return calls

    def extract_tool_calls(self, response_ids: List[int]) -> List[ParsedToolCall]:
        return self.extract_from_text(self.tokenizer.decode(list(response_ids)))
