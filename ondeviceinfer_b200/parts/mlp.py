"""Dense gated feed-forward (ondeviceinfer/layers.py:86-113 of UESlubei/ondeviceinfer)."""

from __future__ import annotations

import torch

from ..config.specs import GatedMLPSpec
from ..weights.tensors import TensorDecl
from .base import Part, register_part
from .linear import gated_linear, linear


class GatedMLP(Part):
    graph_safe = True   # no host work that depends on the step's values: may be captured in a CUDA graph
    takes_lazy_norm = True   # x may be a NormedRows: its first product makes the normed operand itself

    """down(silu(gate(x)) * up(x)).  The gate and up matrices are concatenated at load so
    that one matrix product yields both; the activation is taken in fp32 and rounded once."""

    def __init__(self, spec: GatedMLPSpec) -> None:
        super().__init__(spec)
        if spec.activation != "silu":
            raise ValueError(f"activation {spec.activation!r} is not implemented (silu is)")

    def tensor_decls(self):
        s = self.spec
        return [TensorDecl(s.name("gate"), (s.intermediate_size, s.hidden_size)),
                TensorDecl(s.name("up"), (s.intermediate_size, s.hidden_size)),
                TensorDecl(s.name("down"), (s.hidden_size, s.intermediate_size))]

    def load(self, fetch, runtime) -> None:
        s = self.spec
        self.runtime = runtime
        self.w_gate_up = torch.cat([fetch.matrix(s.name("gate")), fetch.matrix(s.name("up"))], 0)
        self.w_down = fetch.matrix(s.name("down"))

    def forward(self, x, ctx, residual) -> None:
        linear(gated_linear(x, self.w_gate_up), self.w_down, residual=residual, track=ctx)


register_part(GatedMLPSpec, GatedMLP)
