"""Typed configurations, read from each architecture's own config.json keys."""
from .reader import ConfigError, KeyReader, read_config_json
from .llama import LlamaConfig, Llama3RopeScaling
from .fobilorn import FobilornConfig
from .nufolix import NufolixConfig
from .ridopel import RidopelConfig
from .marinex import MarinexConfig
from .presets import preset, preset_names

__all__ = ["ConfigError", "KeyReader", "read_config_json", "LlamaConfig", "Llama3RopeScaling", "FobilornConfig", "NufolixConfig", "RidopelConfig", "MarinexConfig", "preset", "preset_names"]
