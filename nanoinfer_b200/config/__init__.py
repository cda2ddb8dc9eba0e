from .base import ConfigError, ModelConfig, field, read_config_json, architecture_name
from .gpt2 import GPT2Config
from .vadonex import VadonexConfig
from .kemuzen import KemuzenConfig
from .mulavik import MulavikConfig
from .nagilix import NagilixConfig

__all__ = ["ConfigError", "ModelConfig", "field", "read_config_json", "architecture_name", "GPT2Config", "VadonexConfig",
           "MulavikConfig", "KemuzenConfig", "NagilixConfig"]
