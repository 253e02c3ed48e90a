"""RMSNorm (reference: engine/engine.py:107-110, engine/fused.py:152-172)."""
import torch

from ..config.specs import RMSNormSpec
from ..csrc import api
from .base import ParamDecl, Part, register_part


class RMSNorm(Part):
    """y = w * x * rsqrt(mean(x^2) + eps), statistics in float32, weight held in float32."""
    takes_partial = True     # add_forward adds up split-K partial sums (csrc.api.Partial) while it reads them

    def param_decls(self):
        return [ParamDecl("weight", (self.spec.dim,), init="norm", keep_float32=True)]

    def bind(self, tensors):
        self.weight = tensors["weight"].to(torch.float32).contiguous()

    def add_forward(self, h, delta, out, rows=None):
        """h (float32 residual stream) += delta (a tensor, a ``csrc.api.Partial`` or None);
        out = norm(h). ``rows``: only these rows, into out[0..len(rows)), leaving h as it is."""
        api.add_rmsnorm(h, delta, self.weight, self.spec.eps, out, rows)
        return out


register_part(RMSNormSpec, RMSNorm)
