"""Qwen3 dense decoder (``Qwen3ForCausalLM``): its config.json keys and the model built from them.

The reference engine reads six of these keys (engine/engine.py:251-258: num_hidden_layers,
num_attention_heads, num_key_value_heads, head_dim with the hidden_size // heads fallback,
rms_norm_eps, rope_theta) and takes the other sizes from tensor shapes; here every size is a
checked key. ``rope_theta`` is accepted at the top level or under ``rope_parameters`` (both
layouts are written by tools in the wild).
"""
from dataclasses import asdict, dataclass
from typing import Optional

from .base import ConfigError, ModelConfig, get
from .specs import AttentionSpec, GatedMLPSpec, LayerSpec, ModelSpec, RMSNormSpec, RotaryHalfSpec


@dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: Optional[bool] = None   # None: the checkpoint decides (lm_head.weight there or not)
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: Optional[int] = None      # layers with index >= this slide (when sliding is on)

    architecture = "Qwen3ForCausalLM"

    @classmethod
    def from_dict(cls, d):
        archs = d.get("architectures")
        if archs is not None and cls.architecture not in archs:
            raise ConfigError(f"config.json names architectures {archs}, not {cls.architecture}")
        H = get(d, "hidden_size", int, positive=True)
        nh = get(d, "num_attention_heads", int, positive=True)
        nkv = get(d, "num_key_value_heads", int, nh, positive=True)
        hd = get(d, "head_dim", int, None, positive=True)
        if hd is None:
            if H % nh:
                raise ConfigError(f"config.json: no head_dim and hidden_size {H} is not a multiple of {nh} heads")
            hd = H // nh
        if nh % nkv:
            raise ConfigError(f"config.json: {nh} attention heads are not a multiple of {nkv} key/value heads")
        if hd % 2:
            raise ConfigError(f"config.json: head_dim {hd} must be even for rotary position encoding")
        if "rope_theta" in d and d["rope_theta"] is not None:
            theta = get(d, "rope_theta", float, positive=True)
        elif isinstance(d.get("rope_parameters"), dict):
            rp = d["rope_parameters"]
            if rp.get("rope_type", "default") != "default":
                raise ConfigError(f"config.json: rope_type {rp.get('rope_type')!r} is not implemented")
            theta = get(rp, "rope_theta", float, positive=True)
        else:
            raise ConfigError("config.json: required key 'rope_theta' is missing")
        scaling = d.get("rope_scaling")
        if scaling not in (None, {}) and scaling.get("rope_type", scaling.get("type")) != "default":
            raise ConfigError(f"config.json: rope_scaling {scaling!r} is not implemented")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act {act!r} is not implemented (silu only)")
        if d.get("attention_bias", False):
            raise ConfigError("config.json: attention_bias=true is not implemented")
        L = get(d, "num_hidden_layers", int, positive=True)
        use_sw = get(d, "use_sliding_window", bool, False)
        sw = get(d, "sliding_window", int, None, positive=True)
        mwl = get(d, "max_window_layers", int, None)
        if use_sw and sw is None:
            raise ConfigError("config.json: use_sliding_window is set but sliding_window is missing")
        tie = d.get("tie_word_embeddings")
        if tie is not None and not isinstance(tie, bool):
            raise ConfigError(f"config.json: 'tie_word_embeddings' must be true or false, got {tie!r}")
        return cls(
            vocab_size=get(d, "vocab_size", int, positive=True), hidden_size=H,
            intermediate_size=get(d, "intermediate_size", int, positive=True), num_hidden_layers=L,
            num_attention_heads=nh, num_key_value_heads=nkv, head_dim=hd,
            rms_norm_eps=get(d, "rms_norm_eps", float, positive=True), rope_theta=theta,
            max_position_embeddings=get(d, "max_position_embeddings", int, 32768, positive=True),
            tie_word_embeddings=tie, use_sliding_window=use_sw, sliding_window=sw,
            max_window_layers=L if mwl is None else mwl,
        )

    def to_dict(self):
        d = asdict(self)
        d["architectures"] = [self.architecture]
        d["model_type"] = "qwen3"
        d["hidden_act"] = "silu"
        d["attention_bias"] = False
        return d

    def layer_window(self, i):
        if self.use_sliding_window and self.sliding_window is not None and i >= self.max_window_layers:
            return self.sliding_window
        return None

    def to_spec(self):
        """Every layer: RMSNorm -> attention (per-head q/k RMSNorm, rotary over the whole head,
        scale head_dim^-0.5) -> RMSNorm -> SiLU-gated MLP; one eps for all norms
        (reference: engine/engine.py:468-498)."""
        H, hd, eps = self.hidden_size, self.head_dim, self.rms_norm_eps
        layers = []
        for i in range(self.num_hidden_layers):
            layers.append(LayerSpec(
                prefix=f"model.layers.{i}.",
                norm_in=RMSNormSpec(H, eps),
                mixer=AttentionSpec(
                    hidden_size=H, num_heads=self.num_attention_heads, num_kv_heads=self.num_key_value_heads,
                    head_dim=hd, scale=hd ** -0.5, qk_norm=RMSNormSpec(hd, eps),
                    position=RotaryHalfSpec(hd, self.rope_theta), window=self.layer_window(i)),
                norm_post=RMSNormSpec(H, eps),
                feed_forward=GatedMLPSpec(H, self.intermediate_size, "silu"),
            ))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab_size, hidden_size=H, layers=tuple(layers),
            schedule=ModelSpec.identity_schedule(self.num_hidden_layers), final_norm=RMSNormSpec(H, eps),
            tie_embeddings=self.tie_word_embeddings, max_positions=self.max_position_embeddings,
        )
