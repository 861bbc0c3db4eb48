"""YAML loading with Hydra-style composition, usable without Hydra installed.

Supports what the shipped recipes and launch scripts use (reference:
``cli/train_grpo.py:688`` ``@hydra.main(config_path='../configs')``):

* ``--config-name <stem>`` and ``--config-dir <dir>`` command line options,
* a ``defaults:`` list whose entries ``- model: [a, b]`` / ``- model: a`` load
  ``<dir>/model/<a>.yaml`` into the ``model`` section (each file is ``{name: {...}}``),
  and plain strings that merge another top-level YAML first,
* ``section.key=value`` dotted overrides (``+section.key=value`` also accepted),
* ``_self_`` ordering markers are tolerated.

``parse_training_config`` turns the composed dictionary into validated config objects the
same way each ``cli/train_*.py`` of the reference does (``cli/train_grpo.py:227-306``,
``cli/train_ppo.py`` adds ``critic_config``).
"""
from __future__ import annotations

import argparse
import copy
import os
from typing import Any, Dict, List, Optional, Sequence

import yaml

from .rl_options import GenerateConfig, MsprobeConfig, ProfilerConfig, RLConfig
from .training_config import MegatronConfig
from .validate import validate_rl_args

DEFAULT_CONFIG_DIR = os.path.abspath(
    os.path.join(os.path.dirname(__file__), "..", "..", "configs"))


def _deep_merge(dst: Dict[str, Any], src: Dict[str, Any]) -> Dict[str, Any]:
    for k, v in src.items():
        if isinstance(v, dict) and isinstance(dst.get(k), dict):
            _deep_merge(dst[k], v)
        else:
            dst[k] = copy.deepcopy(v)
    return dst


def _read_yaml(path: str) -> Dict[str, Any]:
    with open(path, "r", encoding="utf-8") as fh:
        return yaml.safe_load(fh) or {}


def _find(stem: str, dirs: Sequence[str], sub: str = "") -> str:
    for d in dirs:
        for ext in (".yaml", ".yml"):
            p = os.path.join(d, sub, stem + ext)
            if os.path.isfile(p):
                return p
    raise FileNotFoundError(f"config '{os.path.join(sub, stem)}' not found in {list(dirs)}")


def _parse_scalar(text: str) -> Any:
    try:
        return yaml.safe_load(text)
    except yaml.YAMLError:
        return text


def apply_overrides(cfg: Dict[str, Any], overrides: Sequence[str]) -> Dict[str, Any]:
    for ov in overrides:
        if "=" not in ov:
            raise ValueError(f"override '{ov}' is not of the form key=value")
        key, value = ov.split("=", 1)
        key = key.lstrip("+")
        node = cfg
        parts = key.split(".")
        for p in parts[:-1]:
            node = node.setdefault(p, {})
        node[parts[-1]] = _parse_scalar(value)
    return cfg


def compose(config_name: str, config_dir: Optional[str] = None,
            overrides: Sequence[str] = ()) -> Dict[str, Any]:
    """Load ``config_name`` and resolve its ``defaults`` list into one plain dict."""
    dirs: List[str] = []
    if config_dir:
        dirs.append(os.path.abspath(config_dir))
    dirs.append(DEFAULT_CONFIG_DIR)
    main = _read_yaml(_find(config_name, dirs))
    defaults = main.pop("defaults", []) or []
    out: Dict[str, Any] = {}
    for entry in defaults:
        if entry == "_self_":
            continue
        if isinstance(entry, str):
            _deep_merge(out, compose(entry, config_dir))
            continue
        for group, names in entry.items():
            names = [names] if isinstance(names, str) else list(names or [])
            section = out.setdefault(group, {})
            for name in names:
                _deep_merge(section, _read_yaml(_find(name, dirs, sub=group)))
    _deep_merge(out, main)
    return apply_overrides(out, overrides)


def load_model_catalogue(names: Sequence[str], config_dir: Optional[str] = None) -> Dict[str, Any]:
    """``{name: architecture dict}`` read from ``<config dir>/model/<name>.yaml``."""
    dirs = ([os.path.abspath(config_dir)] if config_dir else []) + [DEFAULT_CONFIG_DIR]
    out: Dict[str, Any] = {}
    for name in names:
        _deep_merge(out, _read_yaml(_find(name, dirs, sub="model")))
    return out


def parse_cli(argv: Optional[Sequence[str]] = None, default_name: Optional[str] = None):
    """Parse ``--config-name/--config-dir`` plus free ``key=value`` overrides."""
    ap = argparse.ArgumentParser(add_help=True)
    ap.add_argument("--config-name", "-cn", default=default_name)
    ap.add_argument("--config-dir", "-cd", default=None)
    ap.add_argument("--config-path", "-cp", default=None)
    args, rest = ap.parse_known_args(argv)
    if args.config_name is None:
        ap.error("--config-name is required")
    overrides = [r for r in rest if "=" in r and not r.startswith("--")]
    return args.config_name, (args.config_dir or args.config_path), overrides


def load_config(argv: Optional[Sequence[str]] = None, default_name: Optional[str] = None):
    name, cdir, overrides = parse_cli(argv, default_name)
    return compose(name, cdir, overrides)


def _role(config: Dict[str, Any], role_key: str) -> MegatronConfig:
    merged = {**(config.get("megatron_training") or {}), **(config.get(role_key) or {})}
    return MegatronConfig(merged, config.get("model"))


def parse_training_config(config: Dict[str, Any], with_critic: bool = False) -> Dict[str, Any]:
    """Composed dict -> ``{actor,ref,reward[,critic]}_config, rl_config, generate_config, ...``."""
    actor_config = _role(config, "actor_config")
    rl_config = RLConfig(config.get("rl_config"))
    if rl_config.use_integrated_worker:
        for banned in ("ref_config", "reward_config"):
            if banned in config:
                raise ValueError(f"{banned} must not be set when use_integrated_worker is on")
        ref_config = reward_config = actor_config
    else:
        ref_config = _role(config, "ref_config")
        reward_config = _role(config, "reward_config")
    critic_config = None
    if with_critic or "critic_config" in config:
        critic_config = _role(config, "critic_config")
    if actor_config.stage == "ray_dapo" and rl_config.use_integrated_worker:
        ref_for_validation = None  # DAPO has no reference model
    else:
        ref_for_validation = ref_config
    generate_config = GenerateConfig(config.get("generate_config"))
    # vision-language runs: architecture (and optionally a rank range) of the vision tower
    vit_config = _role(config, "vit_config") if "vit_config" in config else None
    validate_rl_args(actor_config, ref_for_validation, reward_config, rl_config, generate_config,
                     critic_config=critic_config, vit_config=vit_config)
    prof = config.get("profiler_config") or {}
    profiler_config = {"integrated": ProfilerConfig(prof.get("integrated", {}), role="integrated")}
    msprobe_config = MsprobeConfig(config.get("msprobe_config") or {}, role="integrated")
    out = dict(actor_config=actor_config, ref_config=ref_config, reward_config=reward_config,
               rl_config=rl_config, generate_config=generate_config,
               profiler_config=profiler_config, msprobe_config=msprobe_config)
    if critic_config is not None:
        out["critic_config"] = critic_config
    if vit_config is not None:
        out["vit_config"] = vit_config
    return out
