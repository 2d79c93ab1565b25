"""y = x W^T for the two compute dtypes.

float32: this library's own FMA kernel (no tensor cores, no TF32), residual add fused.
bfloat16: tensor-core matrix product with fp32 accumulation.  The reference leaves every
projection to the vendor library through ``F.linear`` (ondeviceinfer/attention.py:149-157,
ondeviceinfer/layers.py:109-113, ondeviceinfer/model.py:163); the same library call
stands here for shapes the hand-written kernels do not take.
"""

from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops


def linear(x: torch.Tensor, weight: torch.Tensor, *, residual: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """``x`` [tokens, in], ``weight`` [out, in].

    With ``residual`` (fp32 [tokens, out]) the product is added to it in place and
    nothing is returned; otherwise a new [tokens, out] tensor in ``out_dtype`` (default:
    the dtype of ``x``) is returned.
    """
    n, N = x.shape[0], weight.shape[0]
    if x.dtype == torch.float32:
        if residual is not None:
            ops.gemm_f32(x, weight, residual, residual)
            return None
        out = torch.empty((n, N), dtype=torch.float32, device=x.device)
        ops.gemm_f32(x, weight, out)
        return out
    if x.dtype != torch.bfloat16:
        raise ops.KernelError(f"linear takes float32 or bfloat16 activations, not {x.dtype}")
    y = torch.matmul(x, weight.t())
    ops.LAUNCHES["library"] += 1
    if residual is not None:
        ops.residual_add(residual, y)
        return None
    if out_dtype == torch.float32:
        out = torch.empty((n, N), dtype=torch.float32, device=x.device)
        ops.widen(y, out)
        return out
    return y
