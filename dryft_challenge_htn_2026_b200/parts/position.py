"""Rotary position encoding, rotate-half form (reference: engine/engine.py:113-122).

The part owns the angle tables; the rotation itself is fused into the kernel that also
normalises q/k heads and writes the cache, which takes the tables as arguments. Another position
encoding is another part: with ``fused_tables = True`` and ``tables(n)`` (cos, sin [n, dim/2]
float32) if the fused kernel can use it, or with ``apply(qkv, ctx, n_heads, n_kv_heads, head_dim)``
for one that rewrites the q and k heads of the projection rows [tokens, (nh + 2 nkv) * hd] in place
itself; the attention part then runs the fused kernel without rotation. ``apply`` runs before the
cache write and cannot be combined with a per-head q/k norm (which would have to come first): the
attention part refuses that pair."""
import torch

from ..config.specs import RotaryHalfSpec
from .base import Part, register_part


class RotaryHalf(Part):
    fused_tables = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self._n = 0
        self._cos = self._sin = None

    def tables(self, n):
        """cos, sin [>= n, dim/2] float32: angle(p, j) = p * theta^(-2j/dim), computed in float32."""
        if n > self._n:
            n = max(n, 2 * self._n, 256)
            dim, theta = self.spec.dim, self.spec.theta
            inv = 1.0 / (theta ** (torch.arange(0, dim, 2, device=self.rt.device, dtype=torch.float32) / dim))
            ang = torch.outer(torch.arange(n, device=self.rt.device, dtype=torch.float32), inv)
            self._cos, self._sin, self._n = ang.cos().contiguous(), ang.sin().contiguous(), n
        return self._cos, self._sin


register_part(RotaryHalfSpec, RotaryHalf)
