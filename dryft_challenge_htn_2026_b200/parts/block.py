"""Pre-norm residual block: h += mixer(norm_in(h)); h += feed_forward(norm_post(h)).

The residual stream ``h`` is float32. Each add is fused with the norm that follows it, so the
block takes the previous block's not-yet-added output as ``pending`` and returns its own
feed-forward output the same way (the reference fuses the same pair: engine/engine.py:493-495).

A mixer or feed-forward that sets ``fuses_residual = True`` takes part in a further fusion: its
``forward`` gets ``residual=h`` and may add its output into h itself (returning what
``parts.linear.linear`` returned for its last product, a ``csrc.api.Added``), and its input may be
a ``csrc.api.Normed``, a norm that its first product computes while loading. Parts without the
attribute get and return plain tensors.
"""
import torch

from ..config.specs import LayerSpec
from ..csrc import api
from .base import ParamDecl, Part, build_part, register_part
from .norm import RMSNorm


class PreNormBlock(Part):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.norm_in = build_part(spec.norm_in, rt)
        self.mixer = build_part(spec.mixer, rt)
        self.norm_post = build_part(spec.norm_post, rt)
        self.feed_forward = build_part(spec.feed_forward, rt)

    @property
    def SUB(self):
        return self.spec.names

    def param_decls(self):
        out = []
        for attr, pre in self.SUB:
            out += [ParamDecl(pre + p.name, p.shape, p.init, p.keep_float32) for p in getattr(self, attr).param_decls()]
        return out

    def bind(self, tensors):
        for attr, pre in self.SUB:
            getattr(self, attr).bind({k[len(pre):]: v for k, v in tensors.items() if k.startswith(pre)})

    def weights_in_order(self):
        out = []
        for attr, _ in self.SUB:
            fn = getattr(getattr(self, attr), "weights_in_order", None)
            out += fn() if fn else []
        return out

    def cache_requests(self):
        return self.mixer.cache_requests()

    def prepare(self, max_positions):
        for attr, _ in self.SUB:
            fn = getattr(getattr(self, attr), "prepare", None)
            if fn:
                fn(max_positions)

    def forward(self, ctx, h, pending, views, writes=True, a=None):
        """``a``: norm_in(h) if the caller already has it (the embedding kernel makes it for the
        first block). Returns the feed-forward output, still to be added to h."""
        fm = getattr(self.mixer, "fuses_residual", False)
        ff = getattr(self.feed_forward, "fuses_residual", False)
        if a is None:
            a = _add_norm(self.norm_in, h, pending, self.rt.dtype, fm)
        d = self.mixer.forward(ctx, views, a, writes, **({"residual": h} if fm else {}))
        a = _add_norm(self.norm_post, h, d, self.rt.dtype, ff)
        return self.feed_forward.forward(ctx, a, **({"residual": h} if ff else {}))


def _add_norm(norm, h, delta, dtype, may_defer):
    """h += delta, then norm(h). Only RMSNorm knows ``csrc.api.Added`` and can defer; any other
    norm part is called with a tensor (or None when the delta is in h already)."""
    if isinstance(norm, RMSNorm):
        return norm.add_forward(h, delta, dtype, defer=may_defer)
    out = torch.empty((h.shape[0], h.shape[1]), dtype=dtype, device=h.device)
    return norm.add_forward(h, None if isinstance(delta, api.Added) else delta, out)


register_part(LayerSpec, PreNormBlock)
