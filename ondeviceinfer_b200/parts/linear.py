"""y = x W^T for the two compute dtypes, with the epilogues the layers need.

float32: this library's own FMA kernel (no tensor cores, no TF32), residual add fused.

bfloat16, up to 32 tokens (decode and short chunks; ``ODI_OWN_GEMM_MAX_TOKENS`` moves the limit,
the kernel itself takes any number): the hand-written tcgen05 kernel
(``csrc/gemm_tcgen05.cu``): weights streamed by TMA, fp32 accumulators in tensor memory,
the residual add, the fp32 store of logits and the SiLU-gate product fused into its epilogue.

bfloat16, more tokens (prefill): the vendor library's matrix product with fp32
accumulation, as the reference does for every projection through ``F.linear``
(ondeviceinfer/attention.py:149-157, ondeviceinfer/layers.py:109-113,
ondeviceinfer/model.py:163), followed by this library's elementwise kernels.  The same
holds for shapes the tcgen05 kernel refuses (K not a multiple of 8).
"""

from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops

import os

# Measured on B200 on whole captured decode steps at Qwen3-8B sizes (own kernel / library product):
# batch 8: 3.79 / 4.68 ms, batch 16: 4.45 / 4.65 ms, batch 32: 5.39 / 5.42 ms, batch 64: 8.2 / 7.5 ms,
# so the own kernel serves up to 32 tokens by default.
OWN_KERNEL_MAX_TOKENS = int(os.environ.get("ODI_OWN_GEMM_MAX_TOKENS", "32"))


def _own(x: torch.Tensor, weight: torch.Tensor) -> bool:
    return x.shape[0] <= OWN_KERNEL_MAX_TOKENS and ops.gemm_bf16_supported(x, weight)


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
    if _own(x, weight):
        if residual is not None:
            ops.gemm_bf16(x, weight, residual, ops.EPI_RESIDUAL)
            return None
        wide = out_dtype == torch.float32
        out = torch.empty((n, N), dtype=torch.float32 if wide else torch.bfloat16, device=x.device)
        ops.gemm_bf16(x, weight, out, ops.EPI_STORE_F32 if wide else ops.EPI_STORE_BF16)
        return out
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


def gated_linear(x: torch.Tensor, weight_gate_up: torch.Tensor) -> torch.Tensor:
    """silu(x Wg^T) * (x Wu^T) for ``weight_gate_up`` = gate rows followed by up rows."""
    n, I = x.shape[0], weight_gate_up.shape[0] // 2
    act = torch.empty((n, I), dtype=x.dtype, device=x.device)
    if x.dtype == torch.bfloat16 and _own(x, weight_gate_up):
        ops.gemm_bf16(x, weight_gate_up, act, ops.EPI_SWIGLU)
        return act
    ops.silu_mul(linear(x, weight_gate_up), act)
    return act
