"""RMSNorm part (ondeviceinfer/layers.py:9-33 of UESlubei/ondeviceinfer)."""

from __future__ import annotations

import torch

from ..config.specs import RMSNormSpec
from ..kernels import ops
from ..weights.tensors import TensorDecl
from .base import Part, register_part
from .linear import NormedRows


class RMSNorm(Part):
    graph_safe = True   # no host work that depends on the step's values: may be captured in a CUDA graph
    adds = True         # __call__ takes `add`: a pending residual add done in the norm's own pass

    """weight * cast(x * rsqrt(mean(x^2) + eps)): statistics in fp32, cast to the compute
    dtype before the multiplication by the weight."""

    def tensor_decls(self):
        return [TensorDecl(self.spec.weight_name, (self.spec.size,), "one_plus_normal")]

    def load(self, fetch, runtime) -> None:
        self.runtime = runtime
        self.weight = fetch.vector(self.spec.weight_name)

    def lazy(self, x: torch.Tensor, parts: torch.Tensor):
        """The norm of the whole of ``x`` as a :class:`~ondeviceinfer_b200.parts.linear.NormedRows`:
        ``parts`` [pieces, tokens] are sums of squares of pieces of each row, left by the product that
        wrote ``x``.  For a consumer that says ``takes_lazy_norm``."""
        return NormedRows(x, self.weight, self.spec.eps, parts, self.runtime.dtype)

    def __call__(self, x: torch.Tensor, rows=None, add=None) -> torch.Tensor:
        """``add`` (optional, without ``rows``): a product still to be added to ``x``; it is added in place in
        the same pass when the kernel can, else beforehand."""
        n = x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.spec.size), dtype=self.runtime.dtype, device=x.device)
        if add is not None and not (rows is None and ops.rmsnorm_adds(x, self.weight, out, add)):
            ops.residual_add(x, add)
            add = None
        ops.rmsnorm(x, self.weight, self.spec.eps, out, rows, add=add)
        return out


register_part(RMSNormSpec, RMSNorm)
