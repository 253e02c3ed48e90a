"""Typed configuration: part specifications, the model specification built from them, and the
architecture's own config.json reader."""
from .specs import (AttentionSpec, GatedMLPSpec, LayerSpec, ModelSpec, RMSNormSpec, RotaryHalfSpec, ScheduleEntry)
from .base import ConfigError, ModelConfig
from .qwen3 import Qwen3Config

__all__ = ["AttentionSpec", "GatedMLPSpec", "LayerSpec", "ModelSpec", "RMSNormSpec", "RotaryHalfSpec",
           "ScheduleEntry", "ConfigError", "ModelConfig", "Qwen3Config"]
