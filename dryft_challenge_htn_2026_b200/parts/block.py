"""Pre-norm residual block: h += mixer(norm_in(h)); h += feed_forward(norm_post(h)).

The residual stream ``h`` is float32. Each add is fused with the norm that follows it, so the
block takes the previous block's not-yet-added output as ``pending`` and returns its own
feed-forward output the same way (the reference fuses the same pair: engine/engine.py:493-495).
"""
import torch

from ..config.specs import LayerSpec
from .base import ParamDecl, Part, build_part, register_part


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
        if a is None:
            a = self.norm_in.add_forward(h, pending, torch.empty((h.shape[0], h.shape[1]), dtype=self.rt.dtype,
                                                                 device=h.device))
        d = self.mixer.forward(ctx, views, a, writes)
        a = self.norm_post.add_forward(h, d, a)
        return self.feed_forward.forward(ctx, a)


register_part(LayerSpec, PreNormBlock)
