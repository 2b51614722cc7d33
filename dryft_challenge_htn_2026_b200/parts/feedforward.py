"""Dense gated feed-forward: down(silu(gate(x)) * up(x)) (reference: engine/engine.py:137-146,494-495)."""
import math

import torch

from ..config.specs import DenseMLPSpec, GatedMLPSpec
from ..csrc import api
from .base import ParamDecl, Part, register_part
from .linear import SILU, XIELU, linear


class GatedMLP(Part):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        if spec.activation not in ("silu", "gelu_tanh"):
            raise ValueError(f"activation {spec.activation!r} is not implemented (silu, gelu_tanh)")
        # inner sizes that are no multiples of 8 are served too: ``linear`` hands those products to the library and
        # applies the gate with a row kernel behind it

    def param_decls(self):
        s = self.spec
        g, u, d = s.names
        return [ParamDecl(g, (s.intermediate_size, s.hidden_size)), ParamDecl(u, (s.intermediate_size, s.hidden_size)),
                ParamDecl(d, (s.hidden_size, s.intermediate_size))]

    def bind(self, tensors):
        # gate rows then up rows, as the reference fuses them (engine/engine.py:304-306)
        g, u, d = self.spec.names
        self.w_gate_up = torch.cat([tensors.pop(g), tensors.pop(u)], 0).contiguous()
        self.w_down = tensors.pop(d).contiguous()

    def step_weights(self):
        return [self.w_gate_up, self.w_down]

    def forward(self, ctx, a):
        # the activation and the product with the up rows sit in the epilogue of every product kernel
        act = api.GATE_GELU if self.spec.activation == "gelu_tanh" else (0.0, 0.0)
        return linear(linear(a, self.w_gate_up, SILU, act=act), self.w_down, allow_partial=True)


register_part(GatedMLPSpec, GatedMLP)


class DenseMLP(Part):
    """down(act(up(x))) with the xIELU activation: act(z) = ap z^2 + z/2 for z > 0 and
    an (e^z - 1 - z) + z/2 otherwise, ap = softplus(p), an = 1/2 + softplus(q) from the two learned
    numbers of ``act`` (worked out once, in float64, when the tensors are bound). The activation sits in
    the epilogue of the up projection (every product kernel of the library has it as a mode)."""

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        if spec.activation != "xielu":
            raise ValueError(f"activation {spec.activation!r} is not implemented (xielu only)")

    def param_decls(self):
        s = self.spec
        return [ParamDecl("up", (s.intermediate_size, s.hidden_size)), ParamDecl("down", (s.hidden_size, s.intermediate_size)),
                ParamDecl("act", (2,), init="unit", keep_float32=True)]

    def bind(self, tensors):
        self.w_up = tensors.pop("up").contiguous()
        self.w_down = tensors.pop("down").contiguous()
        p, q = (float(x) for x in tensors.pop("act").to(torch.float64).cpu())
        softplus = lambda x: max(x, 0.0) + math.log1p(math.exp(-abs(x)))
        self.alpha_pos, self.alpha_neg = softplus(p), 0.5 + softplus(q)

    def step_weights(self):
        return [self.w_up, self.w_down]

    def forward(self, ctx, a):
        z = linear(a, self.w_up, XIELU, act=(self.alpha_pos, self.alpha_neg))
        return linear(z, self.w_down, allow_partial=True)


register_part(DenseMLPSpec, DenseMLP)
