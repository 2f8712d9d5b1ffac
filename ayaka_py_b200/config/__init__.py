"""Typed configurations: one per architecture (read from its own config.json
keys) and one for the engine."""

from .model import ConfigError, GPT2Config, LuporaxConfig, ModelConfig, RakalixConfig, VedadraConfig
from .engine import EngineConfig

__all__ = ["ConfigError", "ModelConfig", "GPT2Config", "RakalixConfig", "LuporaxConfig", "VedadraConfig", "EngineConfig"]
