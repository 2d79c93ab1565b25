"""y = x W^T for the two compute dtypes, with the epilogues the layers need.

float32: this library's own FMA kernel (no tensor cores, no TF32), residual add fused.

bfloat16, up to 32 tokens (decode and short chunks; ``ODI_OWN_GEMM_MAX_TOKENS`` moves the limit,
the kernel itself takes any number; up to 64 tokens for the logits): the hand-written tcgen05 kernel
(``csrc/gemm_tcgen05.cu``): weights streamed by TMA, fp32 accumulators in tensor memory,
the residual add, the fp32 store of logits and the SiLU-gate product fused into its epilogue.

bfloat16, more tokens (prefill): from about a thousand tokens on the persistent two-CTA tcgen05 kernel
(``csrc/gemm_prefill_tcgen05.cu``) with the SiLU gate or the residual add in its epilogue (see
``PREFILL_GEMM`` below); with fewer tokens the vendor library's matrix product with fp32 accumulation, as
the reference does for every projection through ``F.linear`` (ondeviceinfer/attention.py:149-157,
ondeviceinfer/layers.py:109-113, ondeviceinfer/model.py:163), followed by this library's elementwise
kernels.  The library also takes shapes the tcgen05 kernels refuse (K not a multiple of 8).
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


# The projections of many tokens.  "auto": the persistent two-CTA tcgen05 kernel from 1,024 tokens on for
# the products with a fused epilogue (gate/up with the SiLU gate, output and down projections with the
# residual add) and from 2,048 on for the plain one, else the library's product followed by this library's
# elementwise kernels.  Measured on B200 (Qwen3-8B sizes, us, own / library + elementwise): 1,024 tokens
# gate/up 148 / 141 + 12, down 74 / 70 + 6, q/k/v 45 / 36; 2,048 tokens 273 / 274 + 24, 145 / 133 + 11,
# 70 / 69; 8,192 tokens 1,040 / 1,031 + 96, 558 / 529 + 44, 267 / 270; with fewer tokens there are too
# few tiles for 74 clusters (256 tokens: q/k/v 23 / 12).  "own" / "library" force one of them.
PREFILL_GEMM = os.environ.get("ODI_PREFILL_GEMM", "auto")
PERSISTENT_MIN_TOKENS_FUSED, PERSISTENT_MIN_TOKENS_PLAIN = 1024, 2048


def _persistent(tokens: int, weight: torch.Tensor, x: torch.Tensor, epi: int, biased: bool = False) -> bool:
    n_out = weight.shape[0] // 2 if epi == ops.EPI_SWIGLU else weight.shape[0]
    out_dtype = torch.float32 if epi in (ops.EPI_STORE_F32, ops.EPI_RESIDUAL) else torch.bfloat16
    if PREFILL_GEMM == "library" or not ops.gemm_prefill_supported(x, weight, n_out, out_dtype):
        return False
    if PREFILL_GEMM == "own":
        return True
    fused = biased or epi in (ops.EPI_SWIGLU, ops.EPI_RESIDUAL)      # a bias is a fused epilogue too
    return tokens >= (PERSISTENT_MIN_TOKENS_FUSED if fused else PERSISTENT_MIN_TOKENS_PLAIN)


class NormedRows:
    """``RMSNorm(rows) * weight`` that has not been computed yet.

    A norm part may hand this to the part after it instead of a tensor when the sums of squares of
    the rows are already known (``parts`` [pieces, tokens]: the product that wrote the rows left
    them).  :func:`linear` and :func:`gated_linear` then make the normed operand inside the
    tensor-core kernel, which saves a kernel and a round trip of the activations; ``materialize()``
    gives the ordinary tensor (the stand-alone norm kernel) to anybody else.
    """

    def __init__(self, rows: torch.Tensor, weight: torch.Tensor, eps: float, parts: torch.Tensor,
                 dtype: torch.dtype) -> None:
        self.rows, self.weight, self.eps, self.parts, self.dtype = rows, weight, eps, parts, dtype
        self._tensor: Optional[torch.Tensor] = None

    @property
    def shape(self):
        return self.rows.shape

    @property
    def device(self):
        return self.rows.device

    def materialize(self) -> torch.Tensor:
        if self._tensor is None:
            self._tensor = torch.empty(self.rows.shape, dtype=self.dtype, device=self.rows.device)
            ops.rmsnorm(self.rows, self.weight, self.eps, self._tensor)
        return self._tensor


class UnmergedSplits:
    """The output of a decode attention whose key splits have not been merged yet: ``partial`` holds, per token,
    head and split, the weighted values with their maximum and sum (what ``ops.attention_mma`` leaves with
    ``combine=False``).  :func:`linear` with a residual merges them inside the tensor-core kernel of the
    product (:func:`merge_in_product` says when), which saves the combine kernel and a round trip of the
    activations; ``materialize()`` runs that kernel and gives the ordinary tensor to anybody else."""

    def __init__(self, partial: torch.Tensor, past: torch.Tensor, plan: Optional[torch.Tensor], *, splits: int,
                 heads: int, head_dim: int, dtype: torch.dtype = torch.bfloat16) -> None:
        self.partial, self.past, self.plan = partial, past, plan
        self.splits, self.heads, self.head_dim, self.dtype = splits, heads, head_dim, dtype
        self._tensor: Optional[torch.Tensor] = None

    @property
    def shape(self):
        return (self.past.numel(), self.heads * self.head_dim)

    @property
    def device(self):
        return self.partial.device

    def materialize(self) -> torch.Tensor:
        if self._tensor is None:
            self._tensor = torch.empty(self.shape, dtype=self.dtype, device=self.partial.device)
            ops.attention_mma_combine(self.partial, self._tensor, self.past, nq=self.heads, d=self.head_dim,
                                      splits=self.splits, tiles_per_split=self.plan)
        return self._tensor


# Off by default: measured on B200 on whole captured decode steps it is slower than the combine kernel it saves
# (Qwen3-8B sizes, 2,048-token context, merged in the product / combine kernel: batch 8 3.70 / 3.47 ms a step, batch 1
# 3.54 / 3.02 ms; Qwen3-14B sizes, 16 unequal sequences 6.76 / 6.15 ms; 32B sizes, 8 x 8,192: 15.9 / 13.3 ms).  Every
# CTA of the product merges all tokens over its share of K again, so the partials are read from L2 once per
# tile of output features (32 times at these sizes) by 128 threads a CTA in several dependent round trips, where
# the combine kernel spreads one pass over a block per (token, head).  ODI_MERGE_IN_PRODUCT=1 turns it on.
MERGE_IN_PRODUCT = os.environ.get("ODI_MERGE_IN_PRODUCT", "0") == "1"


def merge_in_product(tokens: int, weight: torch.Tensor, *, splits: int, heads: int, head_dim: int,
                     biased: bool = False) -> bool:
    """Whether :func:`linear` with a residual can take :class:`UnmergedSplits` of these sizes as they are
    (bf16 weights; the few-token tensor-core kernel in a form whose prologue merges the splits)."""
    if not MERGE_IN_PRODUCT or weight.dtype != torch.bfloat16 or weight.shape[1] != heads * head_dim or splits < 2:
        return False
    return (_own_tokens(tokens, weight, biased) and ops.gemm_bf16_supported(weight, weight)
            and ops.gemm_bf16_fuses_merge(tokens, weight.shape[0], weight.shape[1], splits=splits, nq=heads, d=head_dim))


# A product with this many output features (the logits) has tiles enough without K splits, and there the
# own kernel stays ahead up to its widest token tile: 151,936 features x 4,096 at 64 tokens 192 us against
# 208 us for the library's product, which leaves bf16 logits that a further kernel widens (41 us).
TALL_PRODUCT_FEATURES, TALL_PRODUCT_MAX_TOKENS = 32768, 64


def _own_tokens(tokens: int, weight: torch.Tensor, biased: bool = False) -> bool:
    """Whether the few-token tensor-core kernel serves a product of this many tokens.  A product with a bias
    stays with this library's kernels at every width (the bias joins the fp32 product before its one rounding,
    which a library product that returns bf16 cannot offer): this kernel up to where the many-token one takes over."""
    limit = OWN_KERNEL_MAX_TOKENS
    if weight.shape[0] >= TALL_PRODUCT_FEATURES and limit >= 32:
        limit = max(limit, TALL_PRODUCT_MAX_TOKENS)
    if biased and PREFILL_GEMM != "library":
        limit = max(limit, PERSISTENT_MIN_TOKENS_FUSED - 1)
    return tokens <= limit


def _own(x, weight: torch.Tensor, biased: bool = False) -> bool:
    """Whether the few-token tensor-core kernel serves this product: few enough tokens, operands it can map."""
    like = x.rows if isinstance(x, NormedRows) else x
    return _own_tokens(x.shape[0], weight, biased) and ops.gemm_bf16_supported(like, weight)


def _operand(x, weight: torch.Tensor, n_out: int, epi: int):
    """(x, norm) for ops.gemm_bf16: a lazy norm goes into the kernel if its planned form can take it."""
    if not isinstance(x, NormedRows):
        return x, None
    if ops.gemm_bf16_fuses_norm(x.shape[0], n_out, weight.shape[1], epi):
        return None, (x.rows, x.weight, x.parts, x.eps)
    return x.materialize(), None


def linear(x, weight: torch.Tensor, *, bias: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None, track=None) -> Optional[torch.Tensor]:
    """``x`` [tokens, in] (a tensor, :class:`NormedRows` or :class:`UnmergedSplits`), ``weight`` [out, in], ``bias`` None or fp32 [out]
    (added to the fp32 product before it is rounded or added to the residual).

    With ``residual`` (fp32 [tokens, out]) the product is added to it in place and
    nothing is returned; otherwise a new [tokens, out] tensor in ``out_dtype`` (default:
    the dtype of ``x``) is returned.

    ``track`` (the step context) with ``residual``: if the kernel can, it also leaves the sums of
    squares of the rows it wrote, and ``track.residual_sumsq = (residual, parts)`` says so to the
    next norm; otherwise ``track.residual_sumsq`` is set to None.  Whoever passes ``track`` promises
    not to change ``residual`` afterwards.  If ``track.defers_residual_add`` is set (by a block that
    knows how to finish it: see :func:`flush_residual_add`) and the product came from the vendor
    library, the add itself is left to the norm that follows: ``track.pending_residual_add =
    (residual, product)``.
    """
    n, N = x.shape[0], weight.shape[0]
    if track is not None:
        track.residual_sumsq = None
    biased = bias is not None
    if isinstance(x, NormedRows) and not (x.dtype == torch.bfloat16 and _own(x, weight, biased)):
        x = x.materialize()
    if isinstance(x, UnmergedSplits):
        if residual is not None and merge_in_product(n, weight, splits=x.splits, heads=x.heads, head_dim=x.head_dim,
                                                     biased=biased):
            parts = None
            if track is not None and ops.gemm_bf16_gives_sumsq(n, N, weight.shape[1]):
                parts = torch.empty((ops.gemm_bf16_sumsq_parts(N), n), dtype=torch.float32, device=residual.device)
            ops.gemm_bf16(None, weight, residual, ops.EPI_RESIDUAL, sumsq_out=parts, bias=bias,
                          merge=(x.partial, x.past, x.plan, x.splits, x.heads, x.head_dim))
            if parts is not None:
                track.residual_sumsq = (residual, parts)
            return None
        x = x.materialize()
    if x.dtype == torch.float32:
        if residual is not None:
            ops.gemm_f32(x, weight, residual, residual, bias=bias)
            return None
        out = torch.empty((n, N), dtype=torch.float32, device=x.device)
        ops.gemm_f32(x, weight, out, bias=bias)
        return out
    if x.dtype != torch.bfloat16:
        raise ops.KernelError(f"linear takes float32 or bfloat16 activations, not {x.dtype}")
    if _own(x, weight, biased):
        if residual is not None:
            x, norm = _operand(x, weight, N, ops.EPI_RESIDUAL)
            parts = None
            if track is not None and ops.gemm_bf16_gives_sumsq(n, N, weight.shape[1]):
                parts = torch.empty((ops.gemm_bf16_sumsq_parts(N), n), dtype=torch.float32, device=residual.device)
            ops.gemm_bf16(x, weight, residual, ops.EPI_RESIDUAL, norm=norm, sumsq_out=parts, bias=bias)
            if parts is not None:
                track.residual_sumsq = (residual, parts)
            return None
        wide = out_dtype == torch.float32
        epi = ops.EPI_STORE_F32 if wide else ops.EPI_STORE_BF16
        x, norm = _operand(x, weight, N, epi)
        out = torch.empty((n, N), dtype=torch.float32 if wide else torch.bfloat16, device=weight.device)
        ops.gemm_bf16(x, weight, out, epi, norm=norm, bias=bias)
        return out
    if residual is not None and _persistent(n, weight, x, ops.EPI_RESIDUAL, biased):
        ops.gemm_prefill_bf16(x, weight, residual, ops.EPI_RESIDUAL, bias=bias)
        return None
    if residual is None and _persistent(n, weight, x, ops.EPI_STORE_F32 if out_dtype == torch.float32 else ops.EPI_STORE_BF16, biased):
        wide = out_dtype == torch.float32
        out = torch.empty((n, N), dtype=torch.float32 if wide else torch.bfloat16, device=x.device)
        ops.gemm_prefill_bf16(x, weight, out, ops.EPI_STORE_F32 if wide else ops.EPI_STORE_BF16, bias=bias)
        return out
    if residual is None and out_dtype == torch.float32:
        return _wide_product(x, weight, bias)
    y = torch.matmul(x, weight.t())
    ops.LAUNCHES["library"] += 1
    if biased:
        ops.bias_add(y, bias)          # after the library's rounding: only shapes the own kernels refuse come here
    if residual is not None:
        if track is not None and getattr(track, "defers_residual_add", False):
            # the block that set the flag adds `y` in the norm that follows (one pass instead of two)
            track.pending_residual_add = (residual, y)
        else:
            ops.residual_add(residual, y)
        return None
    return y


def flush_residual_add(ctx) -> None:
    """Do a residual add that :func:`linear` left pending on ``ctx`` (nothing if there is none)."""
    pending = getattr(ctx, "pending_residual_add", None)
    if pending is not None:
        ctx.pending_residual_add = None
        ops.residual_add(*pending)


# fp32 results of bf16 operands (the logits) are never rounded to bf16 on the way, whatever the number of rows:
# a vocabulary of 150,000 logits rounded to 8 bits of mantissa ties often, and the first-index argmax would
# then choose by the batch's width.  So beyond the few-token limit they stay with this library's kernels:
# the many-token kernel from WIDE_PERSISTENT_MIN_ROWS rows on, the few-token kernel tile by tile below
# (token tiles of one feature tile run side by side and share the weight tile in L2), and for a K that the
# tensor-core kernels refuse the fp32 kernel on widened operands.
WIDE_PERSISTENT_MIN_ROWS = 256


def _wide_product(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
    n, N = x.shape[0], weight.shape[0]
    out = torch.empty((n, N), dtype=torch.float32, device=x.device)
    if n >= WIDE_PERSISTENT_MIN_ROWS and PREFILL_GEMM != "library" and ops.gemm_prefill_supported(x, weight, N, torch.float32):
        ops.gemm_prefill_bf16(x, weight, out, ops.EPI_STORE_F32, bias=bias)
    elif ops.gemm_bf16_supported(x, weight):
        ops.gemm_bf16(x, weight, out, ops.EPI_STORE_F32, bias=bias)
    else:
        ops.gemm_f32(x.float(), weight.float(), out, bias=bias)
    return out


def _heads_fit(head_dim: int, rot_dim: int, rotated: bool, write_kv: bool) -> bool:
    return head_dim == 128 and write_kv and (not rotated or rot_dim == head_dim)


def heads_in_epilogue(x, weight_qkv: torch.Tensor, *, head_dim: int, rot_dim: int, rotated: bool, write_kv: bool,
                      biased: bool = False) -> bool:
    """Whether :func:`project_heads` can serve this step: a tensor-core kernel in a form whose epilogue
    prepares the heads (bf16, heads of 128, whole-head rotation or none, keys/values written; decode widths
    or the many-token kernel)."""
    if x.dtype != torch.bfloat16 or not _heads_fit(head_dim, rot_dim, rotated, write_kv):
        return False
    if _own(x, weight_qkv, biased):
        return ops.gemm_bf16_fuses_head_prep(x.shape[0], weight_qkv.shape[0], weight_qkv.shape[1], d=head_dim,
                                             rot_dim=rot_dim, rotated=rotated, write_kv=write_kv)
    like = x.rows if isinstance(x, NormedRows) else x
    least = PERSISTENT_MIN_TOKENS_FUSED if biased else PERSISTENT_MIN_TOKENS_PLAIN
    return (PREFILL_GEMM != "library" and x.shape[0] >= least and weight_qkv.shape[0] % 128 == 0
            and ops.gemm_bf16_supported(like, weight_qkv))


def project_heads(x, weight_qkv: torch.Tensor, head_prep, bias: Optional[torch.Tensor] = None) -> None:
    """The q/k/v projections of ``x`` (a tensor or :class:`NormedRows`) with per-head norm, rotation and the
    cache write done in the product's epilogue; ``head_prep`` is the block ``ops.head_prep(None, ...)`` gives."""
    if _own(x, weight_qkv, bias is not None):
        x, norm = _operand(x, weight_qkv, weight_qkv.shape[0], ops.EPI_HEAD_PREP)
        ops.gemm_bf16(x, weight_qkv, None, ops.EPI_HEAD_PREP, norm=norm, head_prep=head_prep, bias=bias)
        return
    if isinstance(x, NormedRows):
        x = x.materialize()
    ops.gemm_prefill_bf16(x, weight_qkv, None, ops.EPI_HEAD_PREP, head_prep=head_prep, bias=bias)


def gated_linear(x, weight_gate_up: torch.Tensor) -> torch.Tensor:
    """silu(x Wg^T) * (x Wu^T) for ``weight_gate_up`` = gate rows followed by up rows."""
    n, I = x.shape[0], weight_gate_up.shape[0] // 2
    act = torch.empty((n, I), dtype=x.dtype, device=x.device)
    if x.dtype == torch.bfloat16 and _own(x, weight_gate_up):
        x, norm = _operand(x, weight_gate_up, I, ops.EPI_SWIGLU)
        ops.gemm_bf16(x, weight_gate_up, act, ops.EPI_SWIGLU, norm=norm)
        return act
    if isinstance(x, NormedRows):
        x = x.materialize()
    if x.dtype == torch.bfloat16 and _persistent(n, weight_gate_up, x, ops.EPI_SWIGLU):
        ops.gemm_prefill_bf16(x, weight_gate_up, act, ops.EPI_SWIGLU)
        return act
    ops.silu_mul(linear(x, weight_gate_up), act)
    return act
