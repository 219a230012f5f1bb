"""Typed configurations read from each architecture's own config.json keys."""
from .base import ConfigError, ModelConfig, load_config, read_json
from .fegarax import FegaraxConfig
from .lakulix import LakulixConfig
from .nirotar import NirotarConfig
from .qwen3 import Qwen3Config
from .vogunex import VogunexConfig

__all__ = ["ConfigError", "FegaraxConfig", "LakulixConfig", "ModelConfig", "NirotarConfig", "Qwen3Config", "VogunexConfig", "load_config", "read_json"]
