"""Parts a model is put together from: norms, position encodings, mixers, feed-forwards, blocks."""
from .base import ParamDecl, Part, Runtime, build_part, register_part
from . import norm, position, attention, feedforward, block  # noqa: F401  (register the built-in parts)
from .attention import GQAAttention
from .block import PreNormBlock
from .feedforward import GatedMLP
from .norm import RMSNorm
from .position import RotaryHalf

__all__ = ["ParamDecl", "Part", "Runtime", "build_part", "register_part", "GQAAttention", "PreNormBlock", "GatedMLP",
           "RMSNorm", "RotaryHalf"]
