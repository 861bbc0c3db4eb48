"""Console / W&B / SwanLab sinks.

``Loggers.info(metrics_dict, iteration, steps)`` prints one formatted line per iteration;
plain strings are passed through.  Unlike the reference (which prints only on the last rank,
``mindspeed_rl/utils/loggers.py:50-56``) the driver decides who logs.
"""
from __future__ import annotations

import logging
import os
import sys
from datetime import datetime
from typing import Any, Dict, Optional


def _fmt(v: Any) -> str:
    if isinstance(v, float):
        return f"{v:.6g}"
    return str(v)


class Loggers:
    def __init__(self, name: str = "mindspeed_rl_b200", logger_level: str = "INFO"):
        self.logger = logging.getLogger(name)
        if not self.logger.handlers:
            h = logging.StreamHandler(sys.stdout)
            h.setFormatter(logging.Formatter("%(asctime)s [%(levelname)s] %(name)s: %(message)s"))
            self.logger.addHandler(h)
            self.logger.propagate = False
        self.logger.setLevel(getattr(logging, logger_level.upper(), logging.INFO))

    def handle_msg(self, msg, level: str, iteration: Optional[int], steps: Optional[int]) -> None:
        if isinstance(msg, dict):
            head = ""
            if iteration is not None:
                head = f"iteration: {iteration}" + (f" / {steps}" if steps is not None else "") + " | "
            text = head + " | ".join(f"{k}: {_fmt(v)}" for k, v in msg.items())
        else:
            text = str(msg)
        getattr(self.logger, level)(text)

    def info(self, msg, iteration=None, steps=None):
        self.handle_msg(msg, "info", iteration, steps)

    def warning(self, msg, iteration=None, steps=None):
        self.handle_msg(msg, "warning", iteration, steps)

    def debug(self, msg, iteration=None, steps=None):
        self.handle_msg(msg, "debug", iteration, steps)

    def error(self, msg, iteration=None, steps=None):
        self.handle_msg(msg, "error", iteration, steps)


class WandbLogger:
    """Weights & Biases sink (``use_wandb``); a missing package or API key disables it."""

    def __init__(self, kwargs: Dict[str, Any]):
        self.run = None
        try:
            import wandb

            os.makedirs(kwargs.get("wandb_save_dir") or "./wandb", exist_ok=True)
            self.run = wandb.init(project=kwargs.get("wandb_project") or "mindspeed_rl_b200",
                                  name=(kwargs.get("wandb_exp_name") or "run") +
                                  datetime.now().strftime("-%m%d-%H%M"),
                                  dir=kwargs.get("wandb_save_dir") or "./wandb",
                                  mode=os.environ.get("WANDB_MODE", "offline"))
            self.wandb = wandb
        except Exception as e:  # pragma: no cover - optional dependency
            print(f"[WandbLogger] disabled: {e}")

    def log_metrics(self, metrics: Dict[str, Any], step: int) -> None:
        if self.run is not None:
            self.wandb.log({k: v for k, v in metrics.items() if isinstance(v, (int, float))}, step=step)


class SwanLabLogger:
    """SwanLab sink (``use_swanlab``); disabled when the package is absent."""

    def __init__(self, kwargs: Dict[str, Any]):
        self.run = None
        try:
            import swanlab  # type: ignore

            self.run = swanlab.init(project=kwargs.get("swanlab_project") or "mindspeed_rl_b200",
                                    experiment_name=kwargs.get("swanlab_exp_name") or "run",
                                    logdir=kwargs.get("swanlab_save_dir") or "./swanlab",
                                    mode=kwargs.get("swanlab_mode") or "local")
            self.swanlab = swanlab
        except Exception as e:  # pragma: no cover - optional dependency
            print(f"[SwanLabLogger] disabled: {e}")

    def log_metrics(self, metrics: Dict[str, Any], step: int) -> None:
        if self.run is not None:
            self.swanlab.log({k: v for k, v in metrics.items() if isinstance(v, (int, float))}, step=step)
