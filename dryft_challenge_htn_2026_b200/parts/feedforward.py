"""Dense gated feed-forward: down(silu(gate(x)) * up(x)) (reference: engine/engine.py:137-146,494-495)."""
import torch

from ..config.specs import GatedMLPSpec
from .base import ParamDecl, Part, register_part
from .linear import SILU, linear


class GatedMLP(Part):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        if spec.activation != "silu":
            raise ValueError(f"activation {spec.activation!r} is not implemented (silu only)")
        if rt.dtype == torch.bfloat16 and (spec.hidden_size % 8 or spec.intermediate_size % 8):
            raise ValueError("bfloat16 products need hidden and intermediate sizes that are multiples of 8, "
                             f"not {spec.hidden_size} / {spec.intermediate_size}")

    def param_decls(self):
        s = self.spec
        return [ParamDecl("gate_proj.weight", (s.intermediate_size, s.hidden_size)),
                ParamDecl("up_proj.weight", (s.intermediate_size, s.hidden_size)),
                ParamDecl("down_proj.weight", (s.hidden_size, s.intermediate_size))]

    def bind(self, tensors):
        # gate rows then up rows, as the reference fuses them (engine/engine.py:304-306)
        self.w_gate_up = torch.cat([tensors.pop("gate_proj.weight"), tensors.pop("up_proj.weight")], 0).contiguous()
        self.w_down = tensors.pop("down_proj.weight").contiguous()

    def step_weights(self):
        return [self.w_gate_up, self.w_down]

    def forward(self, ctx, a):
        return linear(linear(a, self.w_gate_up, SILU), self.w_down, allow_partial=True)


register_part(GatedMLPSpec, GatedMLP)
