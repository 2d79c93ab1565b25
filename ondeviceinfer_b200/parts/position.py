"""Position encodings applied inside a mixer."""

from __future__ import annotations

import torch

from ..config.specs import NoPositionSpec, RotarySpec
from ..kernels import ops
from .base import Part, register_part


class Rotary(Part):
    """Half-split rotary embedding (ondeviceinfer/layers.py:36-83).

    ``inv_freq[i] = 1 / theta**(2i / d)`` is evaluated once on the host in fp32 exactly
    as the reference does (ondeviceinfer/layers.py:44-46); angles, cos and sin of a
    step's positions are evaluated on the device in fp32 and shared by all layers.
    """

    def __init__(self, spec: RotarySpec) -> None:
        super().__init__(spec)
        if spec.dim % 2 != 0 or spec.dim > spec.head_dim or spec.dim <= 0:
            raise ValueError(f"rotary_dim must be even and at most head_dim, got {spec.dim} of {spec.head_dim}")
        self.rot_dim = spec.dim

    def load(self, fetch, runtime) -> None:
        self.runtime = runtime
        exponent = torch.arange(0, self.rot_dim, 2, dtype=torch.float32) / self.rot_dim
        self.inv_freq = (1.0 / (self.spec.theta ** exponent)).to(runtime.device)

    def rotary_tables(self, ctx):
        def make():
            n, half = ctx.n_tokens, self.rot_dim // 2
            cos = torch.empty((n, half), dtype=torch.float32, device=self.inv_freq.device)
            sin = torch.empty_like(cos)
            ops.rope_table(self.inv_freq, ctx.tok_pos, cos, sin)
            return cos, sin

        return ctx.memo(("rotary", self.spec), make)


class NoPosition(Part):
    rot_dim = 0

    def rotary_tables(self, ctx):
        return None


register_part(RotarySpec, Rotary)
register_part(NoPositionSpec, NoPosition)
