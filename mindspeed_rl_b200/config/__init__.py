"""Configuration system: YAML sections -> validated config objects."""
from .schema import ConfigKeyError, SchemaConfig
from .training_config import MegatronConfig, TEMPLATES_DIR
from .rl_options import (DataHandlerConfig, GenerateConfig, MsprobeConfig, ProfilerConfig,
                         RLConfig)
from .validate import get_node_nums, validate_data_handler_config, validate_rl_args
from .loader import (DEFAULT_CONFIG_DIR, apply_overrides, compose, load_config, parse_cli,
                     parse_training_config)

BaseConfig = SchemaConfig

__all__ = [
    "BaseConfig", "SchemaConfig", "ConfigKeyError", "MegatronConfig", "RLConfig",
    "GenerateConfig", "ProfilerConfig", "MsprobeConfig", "DataHandlerConfig",
    "validate_rl_args", "validate_data_handler_config", "get_node_nums", "compose",
    "load_config", "parse_cli", "parse_training_config", "apply_overrides",
    "DEFAULT_CONFIG_DIR", "TEMPLATES_DIR",
]
