"""RMSNorm (reference: engine/engine.py:107-110, engine/fused.py:152-172)."""
import torch

from ..config.specs import RMSNormSpec
from ..csrc import api
from .base import ParamDecl, Part, register_part


class RMSNorm(Part):
    """y = w * x * rsqrt(mean(x^2) + eps), statistics in float32, weight held in float32."""

    def param_decls(self):
        return [ParamDecl("weight", (self.spec.dim,), init="norm", keep_float32=True)]

    def bind(self, tensors):
        self.weight = tensors["weight"].to(torch.float32).contiguous()

    def add_forward(self, h, delta, out, rows=None, defer=False):
        """h (float32 residual stream) += delta; out = norm(h). ``rows``: only these rows, into
        out[0..len(rows)), leaving h as it is. ``delta`` may be a ``csrc.api.Added`` (already in
        h); then, with ``defer``, nothing is launched and a ``csrc.api.Normed`` comes back, which
        the product that consumes it computes on the fly. ``out`` may be a dtype instead of a
        tensor: the output is then allocated when it is needed."""
        lazy = isinstance(delta, api.Added)
        if lazy and defer and rows is None:
            return api.Normed(h, delta.sq, self.weight, self.spec.eps, out if isinstance(out, torch.dtype) else out.dtype)
        if isinstance(out, torch.dtype):
            out = torch.empty((h.shape[0] if rows is None else rows.numel(), h.shape[1]), dtype=out, device=h.device)
        api.add_rmsnorm(h, None if lazy else delta, self.weight, self.spec.eps, out, rows)
        return out


register_part(RMSNormSpec, RMSNorm)
