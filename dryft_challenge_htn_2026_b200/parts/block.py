"""Pre-norm residual block: h += mixer(norm_in(h)); h += feed_forward(norm_post(h)).

The residual stream ``h`` is float32. Each add is fused with the norm that follows it, so the
block takes the previous block's not-yet-added output as ``pending`` and returns its own
feed-forward output the same way (the reference fuses the same pair: engine/engine.py:493-495).
A mixer or feed-forward may return its output as split-K partial sums (``csrc.api.Partial``); a
norm that says ``takes_partial`` adds them up while it reads, for any other they are summed first.
"""
import torch

from ..config.specs import LayerSpec
from ..csrc import api
from .base import ParamDecl, Part, build_part, register_part


class PreNormBlock(Part):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.norm_in = build_part(spec.norm_in, rt)
        self.mixer = build_part(spec.mixer, rt)
        self.norm_post = build_part(spec.norm_post, rt)
        self.feed_forward = build_part(spec.feed_forward, rt)

    def _subparts(self):
        return [(getattr(self, attr), pre) for attr, pre in self.spec.names]

    def param_decls(self):
        return [ParamDecl(pre + p.name, p.shape, p.init, p.keep_float32) for part, pre in self._subparts()
                for p in part.param_decls()]

    def bind(self, tensors):
        for part, pre in self._subparts():
            part.bind({k[len(pre):]: v for k, v in tensors.items() if k.startswith(pre)})

    def step_weights(self):
        """The tensors a step streams once, whatever the batch (for the bytes a decode step must read)."""
        return [w for part, _ in self._subparts() for w in part.step_weights()]

    def step_plans(self):
        return [p for part, _ in self._subparts() for p in part.step_plans()]

    def cache_requests(self):
        return self.mixer.cache_requests()

    def prepare(self, max_positions):
        for part, _ in self._subparts():
            part.prepare(max_positions)

    def forward(self, ctx, h, pending, views, writes=True, a=None):
        """``a``: norm_in(h) if the caller already has it (the embedding kernel makes it for the
        first block). Returns the feed-forward output, still to be added to h."""
        if a is None:
            a = add_norm(self.norm_in, h, pending, self.rt.dtype)
        d = self.mixer.forward(ctx, views, a, writes)
        a = add_norm(self.norm_post, h, d, self.rt.dtype)
        return self.feed_forward.forward(ctx, a)


def add_norm(norm, h, delta, dtype, rows=None):
    """h += delta, then norm(h) (of the rows ``rows`` only, leaving h alone, when given)."""
    if isinstance(delta, api.Partial) and not getattr(norm, "takes_partial", False):
        delta = delta.sum(dtype)
    n = h.shape[0] if rows is None else rows.numel()
    out = torch.empty((n, h.shape[1]), dtype=dtype, device=h.device)
    return norm.add_forward(h, delta, out, rows)


register_part(LayerSpec, PreNormBlock)
