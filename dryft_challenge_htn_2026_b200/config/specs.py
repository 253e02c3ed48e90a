"""Specifications of parts and of a whole model.

A specification is plain data: the sizes and constants a part needs, nothing about the model it
ends up in. An architecture's config class turns its config.json into a ``ModelSpec``; the parts
registry (``parts.registry``) turns each specification into the part that runs it. A new kind of
mixer, feed-forward, norm or position encoding is a new specification class plus a part class
registered for it; nothing in this file has to change.
"""
from dataclasses import dataclass, field
from typing import Any, Optional, Tuple


@dataclass(frozen=True)
class RMSNormSpec:
    """y = w * x * rsqrt(mean(x^2) + eps) over the last ``dim`` elements."""
    dim: int
    eps: float


@dataclass(frozen=True)
class RotaryHalfSpec:
    """Rotate-half rotary encoding over the whole head: angle(p, j) = p * theta^(-2j/dim)."""
    dim: int
    theta: float


@dataclass(frozen=True)
class AttentionSpec:
    """Causal grouped-query softmax attention with q/k/v/o projections without bias."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float                               # multiplies q.k before the softmax
    qk_norm: Optional[Any] = None              # norm spec over head_dim applied to q and k heads
    position: Optional[Any] = None             # position-encoding spec applied to q and k
    window: Optional[int] = None               # keys a query sees, itself included; None: all


@dataclass(frozen=True)
class GatedMLPSpec:
    """down(act(gate(x)) * up(x)) without bias."""
    hidden_size: int
    intermediate_size: int
    activation: str = "silu"


@dataclass(frozen=True)
class LayerSpec:
    """One pre-norm residual block: h += mixer(norm_in(h)); h += feed_forward(norm_post(h)).
    ``prefix`` is the layer's tensor-name prefix in the checkpoint."""
    prefix: str
    norm_in: Any
    mixer: Any
    norm_post: Any
    feed_forward: Any
    # checkpoint name of each sub-part under the prefix
    names: Tuple[Tuple[str, str], ...] = (("norm_in", "input_layernorm."), ("mixer", "self_attn."),
                                          ("norm_post", "post_attention_layernorm."), ("feed_forward", "mlp."))


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer. ``cache`` names the cache entry the layer's mixer uses; with
    ``writes=False`` the mixer only reads what the entry's owner stored in this step."""
    layer: int
    cache: int
    writes: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: Any
    tie_embeddings: Optional[bool]             # None: decided by the checkpoint (lm_head present or not)
    max_positions: int
    embed_name: str = "model.embed_tokens.weight"
    final_norm_prefix: str = "model.norm."
    head_name: str = "lm_head.weight"
    extra: dict = field(default_factory=dict, compare=False)

    @staticmethod
    def identity_schedule(n_layers):
        return tuple(ScheduleEntry(i, i, True) for i in range(n_layers))
