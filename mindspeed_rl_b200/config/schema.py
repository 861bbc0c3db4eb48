"""Declarative config schema machinery.

Every config class of the framework is a *schema* (ordered mapping ``key -> default``)
plus a small amount of post-processing.  ``SchemaConfig.update`` enforces the one rule
users of the YAML surface depend on: a key that is not part of the schema is an error,
``-`` in key names is accepted as ``_``, and a ``model: <name>`` entry pulls in the named
model sub-dictionary *before* the remaining keys are applied, so role keys win over
model keys (reference behaviour: ``mindspeed_rl/config_cls/base_config.py:13-33``).
"""
from __future__ import annotations

import copy
import json
from pathlib import Path
from typing import Any, Dict, Iterable, Mapping, Optional


class ConfigKeyError(ValueError):
    """Raised when a YAML key is not registered in the schema of its section."""


def _unknown(cls_name: str, key: str) -> ConfigKeyError:
    return ConfigKeyError(
        f"{cls_name}: key '{key}' is not a registered option. "
        f"Check the spelling or register it in the schema."
    )


class SchemaConfig:
    """Attribute bag whose legal attribute set is fixed by ``SCHEMA``.

    Sub-classes set ``SCHEMA`` (a dict of defaults, possibly merged from several groups)
    and may override ``_finalize``.
    """

    SCHEMA: Mapping[str, Any] = {}

    def __init__(self, *sources: Optional[Mapping[str, Any]], **kw):
        for key, default in self.SCHEMA.items():
            object.__setattr__(self, key, copy.deepcopy(default))
        self._extra_init(**kw)
        for src in sources:
            if src:
                self.update(src)
        self._finalize()

    # hooks -----------------------------------------------------------------
    def _extra_init(self, **kw) -> None:  # pragma: no cover - trivial
        for k, v in kw.items():
            object.__setattr__(self, k, v)

    def _finalize(self) -> None:
        """Derive dependent values after all sources were applied."""

    # core ------------------------------------------------------------------
    def update(self, config_dict: Mapping[str, Any], model_config_dict=None) -> None:
        if "model" in config_dict:
            if isinstance(model_config_dict, (str, Path)):
                self._apply_multimodal_model(model_config_dict)
            elif model_config_dict is not None:
                name = config_dict["model"]
                if name not in model_config_dict:
                    raise ConfigKeyError(f"model '{name}' not found in the model section")
                self.update(model_config_dict[name])
        for raw_key, value in config_dict.items():
            if raw_key == "model":
                continue
            key = raw_key.replace("-", "_")
            if not hasattr(self, key):
                raise _unknown(type(self).__name__, raw_key)
            setattr(self, key, value)

    def _apply_multimodal_model(self, path) -> None:
        path = Path(path)
        if not path.is_file():
            raise FileNotFoundError(f"multimodal model json not found: {path.absolute()}")
        cfg = json.loads(path.read_text())
        img = cfg.get("image_encoder", {}).get("vision_encoder", {}).get("pipeline_num_layers")
        llm = cfg.get("text_decoder", {}).get("pipeline_num_layers")
        if img is None or llm is None:
            raise ValueError(f"`pipeline_num_layers` must be set in {path}")
        self.num_layer_list = [img, llm]
        self.mm_model = str(path)

    # mapping-like helpers -----------------------------------------------------
    def items(self):
        return self.__dict__.items()

    def dict(self) -> Dict[str, Any]:
        return self.__dict__

    def get(self, key: str, default=None):
        return getattr(self, key, default)

    def keys(self) -> Iterable[str]:
        return self.__dict__.keys()

    def __contains__(self, key: str) -> bool:
        return key in self.__dict__

    def __repr__(self) -> str:
        return f"<{type(self).__name__} {vars(self)}>"


def merge_schemas(*groups: Mapping[str, Any]) -> Dict[str, Any]:
    out: Dict[str, Any] = {}
    for g in groups:
        dup = set(out) & set(g)
        if dup:
            raise RuntimeError(f"duplicate schema keys: {sorted(dup)}")
        out.update(g)
    return out
