"""Python launchers of the CUDA kernels: thin, checked, allocation-free where the caller gives the output.

Every function takes CUDA tensors, checks what the kernel assumes (device, dtype,
contiguity, sizes), launches on the current stream and raises :class:`KernelError`
with the CUDA error text if the launch failed.  There is no CPU path: on a machine
without a GPU, or without the compiled libraries, these functions raise.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import Structure, byref, c_float, c_int, c_long, c_ulonglong, c_void_p
from typing import List, Optional, Sequence, Tuple

import torch

from .build import load_library

ODI_ERR_UNSUPPORTED = 10001
ODI_ERR_ARGUMENT = 10002


class KernelError(RuntimeError):
    pass


def _cuda_error_text(code: int) -> str:
    if code == ODI_ERR_UNSUPPORTED:
        return "the kernel does not take these sizes or this alignment"
    if code == ODI_ERR_ARGUMENT:
        return "inconsistent arguments"
    try:
        rt = ctypes.CDLL("libcudart.so.12")
        rt.cudaGetErrorString.restype = ctypes.c_char_p
        return rt.cudaGetErrorString(code).decode()
    except OSError:
        return f"CUDA error {code}"


# Kernels of this library launched so far in this process (library matrix products are
# counted apart); the benchmark reads the difference over its timed region.
LAUNCHES = {"own": 0, "library": 0}


def _check(code: int, what: str, kernels: int = 1) -> None:
    if code != 0:
        raise KernelError(f"{what}: {_cuda_error_text(code)} (code {code})")
    LAUNCHES["own"] += kernels


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return 0
    if dtype == torch.bfloat16:
        return 1
    raise KernelError(f"kernels take float32 or bfloat16, not {dtype}")


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _require(t: torch.Tensor, name: str, dtype=None, ndim=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (this library has no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise KernelError(f"{name} must have {ndim} dimensions, got shape {tuple(t.shape)}")


# ------------------------------------------------------------------------------ elementwise


def embed(table: torch.Tensor, ids: torch.Tensor, hidden: torch.Tensor) -> None:
    """hidden[t, :] = table[ids[t], :] into the fp32 residual stream."""
    _require(table, "table", ndim=2)
    _require(ids, "ids", torch.int32, 1)
    _require(hidden, "hidden", torch.float32, 2)
    if hidden.shape != (ids.numel(), table.shape[1]):
        raise KernelError(f"hidden is {tuple(hidden.shape)}, expected {(ids.numel(), table.shape[1])}")
    lib = load_library("elementwise")
    _check(lib.odi_embed(_ptr(table), _ptr(ids), _ptr(hidden), c_int(ids.numel()), c_int(table.shape[1]),
                         c_int(dtype_code(table.dtype)), _stream()), "embed")


def rmsnorm_adds(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, add: torch.Tensor) -> bool:
    """Whether :func:`rmsnorm` can take ``add`` for these tensors (the vector form: a width that is a multiple of 4
    and at most 8,192, aligned tensors, ``add`` in the dtype of ``out``)."""
    if add.dtype != out.dtype or add.shape != x.shape or not add.is_contiguous():
        return False
    lib = load_library("elementwise")
    return bool(lib.odi_rmsnorm_adds(_ptr(x), _ptr(weight), _ptr(out), _ptr(add), c_int(x.shape[1])))


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None, add: Optional[torch.Tensor] = None) -> None:
    """out[i] = weight * cast(x[r_i] * rsqrt(mean(x[r_i]^2) + eps)), r_i = rows[i] or i.

    ``add`` ([tokens, H] in the dtype of ``out``, without ``rows``; see :func:`rmsnorm_adds`): first x += add, in
    place, then the norm of the sum: the residual add of a product and the norm after it in one pass."""
    _require(x, "x", torch.float32, 2)
    _require(weight, "weight", torch.float32, 1)
    _require(out, "out", ndim=2)
    n = out.shape[0]
    H = x.shape[1]
    if weight.numel() != H or out.shape[1] != H:
        raise KernelError(f"rmsnorm sizes disagree: x {tuple(x.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    if rows is not None:
        _require(rows, "rows", torch.int32, 1)
        if rows.numel() != n:
            raise KernelError("rows and out disagree")
    elif x.shape[0] != n:
        raise KernelError("x and out disagree")
    if add is not None:
        _require(add, "add", out.dtype, 2)
        if rows is not None or add.shape != x.shape:
            raise KernelError("rmsnorm: add goes without rows and has the shape of x")
    lib = load_library("elementwise")
    _check(lib.odi_rmsnorm(_ptr(x), _ptr(weight), _ptr(out), _ptr(rows), _ptr(add), c_int(n), c_int(H), c_float(eps),
                           c_int(dtype_code(out.dtype)), _stream()), "rmsnorm")


class _HeadPrepArgs(Structure):
    _fields_ = [("qkv", c_void_p), ("q_out", c_void_p), ("k_pool", c_void_p), ("v_pool", c_void_p),
                ("q_norm_w", c_void_p), ("k_norm_w", c_void_p), ("cos_t", c_void_p), ("sin_t", c_void_p),
                ("tok_seq", c_void_p), ("tok_pos", c_void_p), ("page_start", c_void_p), ("page_ids", c_void_p),
                ("n_tokens", c_int), ("nq", c_int), ("nkv", c_int), ("d", c_int), ("rot_dim", c_int),
                ("page_size", c_int), ("ring_pages", c_int), ("write_kv", c_int), ("eps", c_float)]


def rope_table(inv_freq: torch.Tensor, tok_pos: torch.Tensor, cos_t: torch.Tensor, sin_t: torch.Tensor) -> None:
    """cos_t/sin_t[t, i] = cos/sin(tok_pos[t] * inv_freq[i]) in fp32."""
    _require(inv_freq, "inv_freq", torch.float32, 1)
    _require(tok_pos, "tok_pos", torch.int32, 1)
    _require(cos_t, "cos_t", torch.float32, 2)
    _require(sin_t, "sin_t", torch.float32, 2)
    n, half = tok_pos.numel(), inv_freq.numel()
    if cos_t.shape != (n, half) or sin_t.shape != (n, half):
        raise KernelError("rope tables must be [tokens, rot_dim / 2]")
    lib = load_library("elementwise")
    _check(lib.odi_rope_table(_ptr(inv_freq), _ptr(tok_pos), _ptr(cos_t), _ptr(sin_t), c_int(n), c_int(half),
                              _stream()), "rope_table")


def head_prep(qkv, q_out, k_pool, v_pool, q_norm_w, k_norm_w, cos_t, sin_t, tok_seq, tok_pos, page_start,
              page_ids, *, nq: int, nkv: int, d: int, rot_dim: int, page_size: int, ring_pages: int,
              write_kv: bool, eps: float) -> None:
    """Per-head Q/K RMSNorm (optional), rotary embedding (optional) and cache write, fused.

    With ``qkv=None`` nothing runs: the checked argument block is returned, for the tensor-core product
    that does the same in its epilogue (``gemm_bf16(..., EPI_HEAD_PREP, head_prep=...)``; bf16 only)."""
    _require(q_out, "q_out", torch.bfloat16 if qkv is None else qkv.dtype, 2)
    n = q_out.shape[0]
    if qkv is not None:
        _require(qkv, "qkv", ndim=2)
        if qkv.shape[0] != n or qkv.shape[1] != (nq + 2 * nkv) * d:
            raise KernelError(f"head_prep sizes disagree: qkv {tuple(qkv.shape)}, nq={nq}, nkv={nkv}, d={d}")
    if q_out.numel() != n * nq * d:
        raise KernelError(f"head_prep sizes disagree: q_out {tuple(q_out.shape)}, nq={nq}, d={d}")
    if write_kv:
        _require(k_pool, "k_pool", q_out.dtype)
        _require(v_pool, "v_pool", q_out.dtype)
    for name, w in (("q_norm_w", q_norm_w), ("k_norm_w", k_norm_w)):
        if w is not None:
            _require(w, name, torch.float32, 1)
            if w.numel() != d:
                raise KernelError(f"{name} has {w.numel()} entries, head_dim is {d}")
    if cos_t is not None:
        _require(cos_t, "cos_t", torch.float32, 2)
        _require(sin_t, "sin_t", torch.float32, 2)
        if cos_t.shape != (n, rot_dim // 2) or sin_t.shape != cos_t.shape:
            raise KernelError("rope tables must be [tokens, rot_dim / 2]")
    args = _HeadPrepArgs(_ptr(qkv), _ptr(q_out), _ptr(k_pool), _ptr(v_pool), _ptr(q_norm_w), _ptr(k_norm_w),
                         _ptr(cos_t), _ptr(sin_t), _ptr(tok_seq), _ptr(tok_pos), _ptr(page_start), _ptr(page_ids),
                         n, nq, nkv, d, rot_dim, page_size, ring_pages, 1 if write_kv else 0, eps)
    if qkv is None:
        return args
    lib = load_library("elementwise")
    _check(lib.odi_head_prep(byref(args), c_int(dtype_code(qkv.dtype)), _stream()), "head_prep")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out = silu(gate_up[:, :I]) * gate_up[:, I:]."""
    _require(gate_up, "gate_up", ndim=2)
    _require(out, "out", gate_up.dtype, 2)
    n, I = out.shape
    if gate_up.shape != (n, 2 * I):
        raise KernelError(f"silu_mul sizes disagree: {tuple(gate_up.shape)} -> {tuple(out.shape)}")
    lib = load_library("elementwise")
    _check(lib.odi_silu_mul(_ptr(gate_up), _ptr(out), c_int(n), c_int(I), c_int(dtype_code(out.dtype)), _stream()),
           "silu_mul")


def residual_add(hidden: torch.Tensor, y: torch.Tensor) -> None:
    """hidden (fp32) += y."""
    _require(hidden, "hidden", torch.float32)
    _require(y, "y")
    if hidden.numel() != y.numel():
        raise KernelError("residual_add sizes disagree")
    lib = load_library("elementwise")
    _check(lib.odi_residual_add(_ptr(hidden), _ptr(y), c_long(hidden.numel()), c_int(dtype_code(y.dtype)), _stream()),
           "residual_add")


def bias_add(y: torch.Tensor, bias: torch.Tensor) -> None:
    """y[t, n] += bias[n] in place (y bf16 or fp32, bias fp32), rounded once to the dtype of y.  For the
    products that the tensor-core kernels refuse and the vendor library computes."""
    _require(y, "y", ndim=2)
    _require_bias(bias, y.shape[1])
    lib = load_library("elementwise")
    _check(lib.odi_bias_add(_ptr(y), _ptr(bias), c_long(y.shape[0]), c_int(y.shape[1]), c_int(dtype_code(y.dtype)),
                            _stream()), "bias_add")


def widen(x: torch.Tensor, out: torch.Tensor) -> None:
    _require(x, "x", torch.bfloat16)
    _require(out, "out", torch.float32)
    lib = load_library("elementwise")
    _check(lib.odi_widen(_ptr(x), _ptr(out), c_long(x.numel()), _stream()), "widen")


# ------------------------------------------------------------------------------ matrix products


def _require_bias(bias: Optional[torch.Tensor], rows: int) -> None:
    if bias is not None:
        _require(bias, "bias", torch.float32, 1)
        if bias.numel() != rows:
            raise KernelError(f"bias has {bias.numel()} entries, the weight has {rows} rows")


def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, residual: Optional[torch.Tensor] = None,
             bias: Optional[torch.Tensor] = None) -> None:
    """out[M,N] = a[M,K] w[N,K]^T (+ bias[N]) (+ residual) in true fp32; residual may be ``out`` itself."""
    _require(a, "a", torch.float32, 2)
    _require(w, "w", torch.float32, 2)
    _require(out, "out", torch.float32, 2)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"gemm sizes disagree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if residual is not None:
        _require(residual, "residual", torch.float32, 2)
        if residual.shape != out.shape:
            raise KernelError("residual and out disagree")
    _require_bias(bias, N)
    lib = load_library("gemm_f32")
    _check(lib.odi_gemm_f32(_ptr(a), _ptr(w), _ptr(out), _ptr(residual), _ptr(bias), c_int(M), c_int(N), c_int(K),
                            c_int(K), c_int(K), c_int(N), c_int(N), _stream()), "gemm_f32")


EPI_STORE_BF16, EPI_STORE_F32, EPI_RESIDUAL, EPI_SWIGLU, EPI_HEAD_PREP = 0, 1, 2, 3, 4

_gemm_state = {}

# Scratch that the wrappers keep per device is handed to kernels by address, and a captured CUDA graph keeps
# replaying with the address it saw.  So a buffer that has to grow is not freed: it is put aside here for
# the life of the process, where a graph that still writes to it does no harm.
_outgrown = []


def _gemm_buffers(device, scratch_floats: int):
    """Scratch for split partials, tile tickets (kept zero between launches) and the error word."""
    device = torch.device(device)
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    state = _gemm_state.setdefault(device, {})
    if "tickets" not in state:
        state["tickets"] = torch.zeros(16384, dtype=torch.int32, device=device)
        state["status"] = torch.zeros(4, dtype=torch.int32, device=device)
        state["scratch"] = torch.empty(1 << 22, dtype=torch.float32, device=device)
    if state["scratch"].numel() < scratch_floats:
        _outgrown.append(state["scratch"])
        state["scratch"] = torch.empty(int(scratch_floats * 1.25), dtype=torch.float32, device=device)
    return state["scratch"], state["tickets"], state["status"]


def kernel_status_word(device) -> torch.Tensor:
    """The error word of the kernels that wait on barriers, as a one-element int32 tensor on ``device``
    (0 = fine).  Whoever already copies a step's result to the host can take it along and call
    :func:`raise_on_kernel_fault` when it is not zero."""
    _, _, status = _gemm_buffers(torch.device(device), 0)
    return status[:1]


def gemm_status(device=None) -> int:
    """The error word of the tensor-core GEMM (0 = fine); reading it synchronises the device."""
    codes = [int(s["status"][0].item()) for d, s in _gemm_state.items() if "status" in s and (device is None or d == device)]
    return next((c for c in codes if c), 0)


def raise_on_kernel_fault() -> None:
    code = gemm_status()
    if code:
        names = {1: "gemm_tcgen05: the TMA producer", 2: "gemm_tcgen05: the MMA issuer", 3: "gemm_tcgen05: the epilogue",
                 21: "gemm_prefill_tcgen05: the TMA producer", 22: "gemm_prefill_tcgen05: the MMA issuer",
                 23: "gemm_prefill_tcgen05: the epilogue",
                 11: "attention_tcgen05: the TMA producer", 12: "attention_tcgen05: the MMA issuer",
                 13: "attention_tcgen05: the softmax warps",
                 31: "attention_mma (decode, TMA-fed): the TMA producer", 32: "attention_mma (decode, TMA-fed): a compute warp"}
        for state in _gemm_state.values():
            state["status"].zero_()
        if code == 33:
            raise KernelError("attention_mma (decode): the host's list of key blocks ends before a sequence's keys do "
                              "(the lengths on the device are not those the list was made for); its result is invalid")
        raise KernelError(f"a kernel gave up waiting on a barrier ({names.get(code, code)}); its result is invalid")


# Token tile for 33 to 64 tokens: 64 (one tile), or 32 (two tiles side by side, which keep the norm prologue,
# the head preparation and the sums of squares that only tiles up to 32 have).
TILE_ABOVE_32 = int(os.environ.get("ODI_GEMM_TILE_ABOVE_32", "64"))


def gemm_bf16_plan(tokens: int, n_out: int, K: int, epi: int):
    """(tile, splits) for a shape: tiles of 128 features x `tile` tokens, with enough K splits for about
    384 CTAs (at most 8, a cluster), each split at least four k-blocks of 64."""
    total_kb = -(-K // 64)
    bn = next((b for b in (16, 32) if tokens <= b), TILE_ABOVE_32 if tokens <= 64 else 64)
    tiles = -(-n_out // 128) * -(-tokens // bn)
    # measured on whole decode steps on B200: about 384 CTAs (three of 72 KB per SM) stream best,
    # in clusters of up to 8 splits (192: +7 %, 288: +2 %, 512: +7 % step time)
    target = 384
    splits = max(1, min(total_kb // 4, int(target / tiles + 0.5), 8)) if tiles < target else 1
    return bn, splits


def gemm_bf16_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    K = x.shape[1]
    return K % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0


def gemm_bf16_sumsq_parts(n_out: int) -> int:
    """Rows of the ``sumsq_out`` a residual product over ``n_out`` features fills: one per tile of 128."""
    return -(-n_out // 128)


def gemm_bf16_fuses_norm(tokens: int, n_out: int, K: int, epi: int) -> bool:
    """Whether the planned form of this product can take its operand through the norm prologue."""
    bn, _ = gemm_bf16_plan(tokens, n_out, K, epi)
    return bn <= 32 and tokens <= 64 and epi in (EPI_STORE_BF16, EPI_SWIGLU, EPI_HEAD_PREP)


def gemm_bf16_fuses_head_prep(tokens: int, n_out: int, K: int, *, d: int, rot_dim: int, rotated: bool,
                              write_kv: bool) -> bool:
    """Whether the planned form of the q/k/v product can prepare the heads in its epilogue: heads of 128
    (a tile of the product is a head), whole-head rotation or none, keys and values written, decode widths."""
    bn, splits = gemm_bf16_plan(tokens, n_out, K, EPI_STORE_BF16)
    return (bn <= 32 and tokens <= 64 and splits <= 8 and d == 128 and n_out % 128 == 0 and write_kv
            and (not rotated or rot_dim == d))


MERGE_SMEM_LIMIT = 96 * 1024


def gemm_bf16_fuses_merge(tokens: int, n_out: int, K: int, *, splits: int, nq: int, d: int) -> bool:
    """Whether the planned form of this residual product can take the unmerged splits of a decode attention
    (``splits`` partials per token and head, ``nq`` heads of ``d``) as its operand: decode widths, heads of a
    multiple of 64, K all the heads, and shared memory for the token tiles of a CTA's share of K."""
    bn, k_splits = gemm_bf16_plan(tokens, n_out, K, EPI_RESIDUAL)
    if bn > 32 or tokens > 64 or k_splits > 8 or not 1 <= splits <= 32 or d % 64 or nq * d != K:
        return False
    kb_cap = -(-(K // 64) // k_splits)
    heads = -(-kb_cap * 64 // d) + 1
    smem = 3 * 128 * 64 * 2 + 1024 + kb_cap * bn * 64 * 2 + bn * heads * (splits + 2) * 4
    return smem <= MERGE_SMEM_LIMIT


class _MergeArgs(Structure):
    _fields_ = [("partial", c_void_p), ("past", c_void_p), ("plan", c_void_p), ("splits", c_int), ("nq", c_int),
                ("d", c_int)]


def gemm_bf16_gives_sumsq(tokens: int, n_out: int, K: int) -> bool:
    """Whether the planned form of this residual product can leave the rows' sums of squares."""
    bn, splits = gemm_bf16_plan(tokens, n_out, K, EPI_RESIDUAL)
    return bn <= 64 and splits <= 8


def gemm_bf16(x: Optional[torch.Tensor], w: torch.Tensor, out: Optional[torch.Tensor], epi: int, *,
              bn: Optional[int] = None, splits: Optional[int] = None, cluster: bool = True,
              norm: Optional[tuple] = None, sumsq_out: Optional[torch.Tensor] = None, head_prep=None,
              bias: Optional[torch.Tensor] = None, merge: Optional[tuple] = None) -> None:
    """Tensor-core product out = epilogue(x w^T): x [tokens, K] bf16, w [rows, K] bf16.

    ``EPI_STORE_BF16`` / ``EPI_STORE_F32``: out [tokens, rows]; ``EPI_RESIDUAL``: out (fp32) += product;
    ``EPI_SWIGLU``: w holds the gate rows then the up rows, out [tokens, rows / 2] = silu(gate) * up.
    ``cluster``: let 2..8 K splits exchange their partials inside a thread-block cluster (else, and for
    more splits, through global scratch and a ticket).
    ``norm = (rows, weight, parts, eps)`` instead of ``x``: the operand is RMSNorm(rows) * weight with the
    roundings of :func:`rmsnorm`, made inside the kernel from the fp32 ``rows`` [tokens, K]; ``parts``
    [pieces, tokens] holds sums of squares of pieces of each row (what ``sumsq_out`` of the product that
    wrote the rows received).  Decode form only (``gemm_bf16_fuses_norm``).
    ``sumsq_out`` (fp32 [gemm_bf16_sumsq_parts(features), tokens]) with ``EPI_RESIDUAL``: receives, per tile
    of 128 features, the sums of squares of the rows the product leaves in ``out``.
    ``EPI_HEAD_PREP`` with ``head_prep`` (the block that ``head_prep(None, ...)`` returns) and ``out=None``:
    w holds query, key and value heads of 128 rows each; the epilogue rounds the projections to bf16 and
    does what :func:`head_prep` does with them (``gemm_bf16_fuses_head_prep`` says when).
    ``bias`` (fp32, one per row of w): added to the fp32 product before the epilogue's own work and rounding.
    ``merge = (partial, past, plan, splits, nq, d)`` instead of ``x``, with ``EPI_RESIDUAL``: the operand is the
    output of a decode attention whose ``splits`` partials per token and head are still apart in ``partial``
    (:func:`attention_mma` with ``combine=False``; ``plan``: its ``tiles_per_split`` or None); the kernel merges
    them as the combine kernel would, bit for bit (``gemm_bf16_fuses_merge`` says when it can).
    """
    merge_args = None
    if merge is not None:
        if x is not None or norm is not None or epi != EPI_RESIDUAL:
            raise KernelError("gemm_bf16 takes merge instead of x and norm, with EPI_RESIDUAL")
        partial, past, plan, m_splits, m_nq, m_d = merge
        _require(partial, "merge partial", torch.float32)
        _require(past, "merge past", torch.int32, 1)
        if plan is not None:
            _require(plan, "merge plan", torch.int32, 1)
        tokens = past.numel()
        if partial.numel() < tokens * m_nq * m_splits * (m_d + 2):
            raise KernelError("merge partial is smaller than tokens x heads x splits x (d + 2)")
        if not gemm_bf16_fuses_merge(tokens, w.shape[0], m_nq * m_d, splits=m_splits, nq=m_nq, d=m_d):
            raise KernelError("this product cannot take unmerged attention splits (see gemm_bf16_fuses_merge)")
        merge_args = _MergeArgs(_ptr(partial), _ptr(past), _ptr(plan), m_splits, m_nq, m_d)
        x_like = torch.empty((tokens, m_nq * m_d), dtype=torch.bfloat16, device="meta")
    if norm is not None:
        if x is not None:
            raise KernelError("gemm_bf16 takes either x or norm")
        rows, norm_w, parts, eps = norm
        _require(rows, "norm rows", torch.float32, 2)
        _require(norm_w, "norm weight", torch.float32, 1)
        _require(parts, "norm parts", torch.float32, 2)
        if norm_w.numel() != rows.shape[1] or parts.shape[1] != rows.shape[0]:
            raise KernelError(f"norm operands disagree: rows {tuple(rows.shape)}, weight {tuple(norm_w.shape)}, "
                              f"parts {tuple(parts.shape)}")
        x_like = rows
    elif merge is None:
        _require(x, "x", torch.bfloat16, 2)
        x_like = x
    _require(w, "w", torch.bfloat16, 2)
    tokens, K = x_like.shape
    w_rows = w.shape[0]
    n_out = w_rows // 2 if epi == EPI_SWIGLU else w_rows
    if epi == EPI_HEAD_PREP:
        if out is not None or head_prep is None:
            raise KernelError("EPI_HEAD_PREP takes head_prep and no out")
        if w.shape[1] != K:
            raise KernelError(f"gemm sizes disagree: x {tuple(x_like.shape)}, w {tuple(w.shape)}")
    else:
        _require(out, "out", torch.bfloat16 if epi in (EPI_STORE_BF16, EPI_SWIGLU) else torch.float32, 2)
        if w.shape[1] != K or out.shape != (tokens, n_out) or (epi == EPI_SWIGLU and w_rows % 2):
            raise KernelError(f"gemm sizes disagree: x {tuple(x_like.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if sumsq_out is not None:
        _require(sumsq_out, "sumsq_out", torch.float32, 2)
        if epi != EPI_RESIDUAL or sumsq_out.shape != (gemm_bf16_sumsq_parts(n_out), tokens):
            raise KernelError("sumsq_out goes with EPI_RESIDUAL and has one row per tile of 128 features")
    if not gemm_bf16_supported(w if merge is not None else x_like, w):
        raise KernelError(f"gemm_tcgen05 needs K a multiple of 8 and 16-byte aligned operands (K={K})")
    _require_bias(bias, w_rows)
    plan_bn, plan_splits = gemm_bf16_plan(tokens, n_out, K, epi)
    bn = plan_bn if bn is None else bn
    splits = plan_splits if splits is None else splits
    lib = load_library("gemm_tcgen05")
    lib.odi_gemm_bf16_scratch_floats.restype = c_long
    need = lib.odi_gemm_bf16_scratch_floats(c_int(tokens), c_int(n_out), c_int(bn), c_int(splits),
                                            c_int(1 if epi == EPI_SWIGLU else 0))
    tiles = -(-n_out // 128) * -(-tokens // bn)
    scratch, tickets, status = _gemm_buffers(w.device, need)
    if splits > 1 and tiles > tickets.numel() // 2:      # the upper half belongs to the many-token kernel's tile flags
        raise KernelError("too many tiles for a split product")
    if norm is not None:
        norm_args = (_ptr(norm[0]), _ptr(norm[1]), _ptr(norm[2]), c_int(norm[2].shape[0]), c_float(norm[3]))
    else:
        norm_args = (_ptr(None), _ptr(None), _ptr(None), c_int(0), c_float(0.0))
    _check(lib.odi_gemm_bf16(_ptr(x), _ptr(w), _ptr(out), c_int(tokens), c_int(n_out), c_int(K), c_int(w_rows),
                             c_int(n_out), c_int(epi), c_int(bn), c_int(splits), c_int(1 if cluster else 0), _ptr(scratch), _ptr(tickets), _ptr(status), *norm_args,
                             _ptr(sumsq_out), byref(head_prep) if head_prep is not None else _ptr(None), _ptr(bias),
                             c_int(0), byref(merge_args) if merge_args is not None else _ptr(None), _stream()),
           "gemm_tcgen05")


SELFTEST_WAIT_CYCLES = 20_000_000        # about ten milliseconds of SM clock


def selftest_bounded_wait(device="cuda:0") -> int:
    """Make one wait of the tensor-core GEMM run out, safely, and return the code the kernel recorded.

    One tile is launched from a build of ``gemm_tcgen05.cu`` whose waits last about ten milliseconds
    (``ODI_WAIT_CYCLES``) with a producer that requests no copy at all, so nothing is in flight: the MMA role
    gives up on its first wait, every role leaves its loop, tensor memory is freed and the kernel returns.
    The error word then holds the MMA role's code (2) and :func:`raise_on_kernel_fault` raises naming it.
    The product's own build and its two-second limit are not involved."""
    device = torch.device(device)
    x = torch.zeros((16, 256), dtype=torch.bfloat16, device=device)
    w = torch.zeros((128, 256), dtype=torch.bfloat16, device=device)
    out = torch.zeros((16, 128), dtype=torch.float32, device=device)
    scratch, tickets, status = _gemm_buffers(device, 0)
    lib = load_library("gemm_tcgen05", {"ODI_WAIT_CYCLES": SELFTEST_WAIT_CYCLES})
    none = _ptr(None)
    with torch.cuda.device(device):
        _check(lib.odi_gemm_bf16(_ptr(x), _ptr(w), _ptr(out), c_int(16), c_int(128), c_int(256), c_int(128), c_int(128),
                                 c_int(EPI_STORE_F32), c_int(16), c_int(1), c_int(0), _ptr(scratch), _ptr(tickets),
                                 _ptr(status), none, none, none, c_int(0), c_float(0.0), none, none, none, c_int(1),
                                 none, _stream()), "gemm_tcgen05 (bounded-wait self-test)")
        torch.cuda.synchronize(device)
    return int(status[0].item())


def gemm_prefill_supported(x: torch.Tensor, w: torch.Tensor, n_out: int, out_dtype: torch.dtype) -> bool:
    """Whether :func:`gemm_prefill_bf16` takes these operands: K a multiple of 8, 16-byte aligned operands, and
    output rows that start on 16-byte boundaries (they leave through TMA stores)."""
    elem = 4 if out_dtype == torch.float32 else 2
    return gemm_bf16_supported(x, w) and (n_out * elem) % 16 == 0


PREFILL_BALANCE = int(os.environ.get("ODI_PREFILL_BALANCE", "1"))     # 0 whole tiles, 1 parts when they pay, 2..4 that many


def gemm_prefill_bf16(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor], epi: int, *, head_prep=None,
                      bias: Optional[torch.Tensor] = None, balance: Optional[int] = None) -> None:
    """The persistent two-CTA tensor-core product for many tokens (``csrc/gemm_prefill_tcgen05.cu``): clusters
    of two CTAs own tiles of 256 tokens x 256 features (tcgen05.mma.cta_group::2), two accumulators in tensor
    memory so that a tile's epilogue runs under the next tile's MMAs, output by TMA store or fp32 reduce-add.
    ``balance`` (default ``ODI_PREFILL_BALANCE``, 1): with ``EPI_RESIDUAL``, cut every tile's k-blocks into up to four
    parts that different CTA pairs add into the residual, in a fixed order, when that shortens the walk (128 tiles
    on 74 pairs: two rounds whole, 1.75 in quarters); 0 whole tiles always, 2..4 that many parts.
    Same operands and epilogues as :func:`gemm_bf16`; with ``EPI_HEAD_PREP`` (``out=None``, ``head_prep`` the block
    that ``head_prep(None, ...)`` returns) a thread of the epilogue finishes a token's row of a head."""
    _require(x, "x", torch.bfloat16, 2)
    _require(w, "w", torch.bfloat16, 2)
    tokens, K = x.shape
    w_rows = w.shape[0]
    n_out = w_rows // 2 if epi == EPI_SWIGLU else w_rows
    if epi == EPI_HEAD_PREP:
        if out is not None or head_prep is None or w.shape[1] != K:
            raise KernelError("EPI_HEAD_PREP takes head_prep, no out, and weights as wide as x")
        if not gemm_bf16_supported(x, w):
            raise KernelError(f"gemm_prefill_tcgen05 needs K a multiple of 8 and 16-byte aligned operands (K={K})")
    else:
        if epi not in (EPI_STORE_BF16, EPI_STORE_F32, EPI_RESIDUAL, EPI_SWIGLU):
            raise KernelError(f"gemm_prefill_bf16 has no epilogue {epi}")
        _require(out, "out", torch.bfloat16 if epi in (EPI_STORE_BF16, EPI_SWIGLU) else torch.float32, 2)
        if w.shape[1] != K or out.shape != (tokens, n_out) or (epi == EPI_SWIGLU and w_rows % 2):
            raise KernelError(f"gemm sizes disagree: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
        if not gemm_prefill_supported(x, w, n_out, out.dtype):
            raise KernelError(f"gemm_prefill_tcgen05 needs K a multiple of 8, 16-byte aligned operands and output rows "
                              f"(K={K}, {n_out} {out.dtype} per row)")
    _require_bias(bias, w_rows)
    _, tickets, status = _gemm_buffers(w.device, 0)
    # the upper half of the ticket array serves as the tiles' flags (the few-token kernel counts tiles in the lower)
    flags = tickets[tickets.numel() // 2:]
    lib = load_library("gemm_prefill_tcgen05")
    _check(lib.odi_gemm_prefill_bf16(_ptr(x), _ptr(w), _ptr(out), c_int(tokens), c_int(n_out), c_int(K), c_int(w_rows),
                                     c_int(n_out), c_int(epi), byref(head_prep) if head_prep is not None else _ptr(None),
                                     _ptr(bias), _ptr(status), _ptr(flags), c_int(flags.numel()),
                                     c_int(PREFILL_BALANCE if balance is None else balance), _stream()),
           "gemm_prefill_tcgen05")


# ------------------------------------------------------------------------------ attention


class _AttnArgs(Structure):
    _fields_ = [("q", c_void_p), ("k_pool", c_void_p), ("v_pool", c_void_p), ("out", c_void_p),
                ("partial", c_void_p), ("cu_q", c_void_p), ("past", c_void_p), ("page_start", c_void_p),
                ("page_ids", c_void_p), ("n_seqs", c_int), ("nq", c_int), ("nkv", c_int), ("page_size", c_int),
                ("ring_pages", c_int), ("window", c_int), ("splits", c_int), ("bq", c_int),
                ("head_chunks", c_int), ("scale", c_float)]


SIMT_HEAD_DIMS = tuple(range(16, 513, 16))


def attention_simt(q, k_pool, v_pool, out, cu_q, past, page_start, page_ids, *, n_seqs: int, max_q_len: int,
                   nq: int, nkv: int, d: int, page_size: int, ring_pages: int, window: int, scale: float,
                   splits: int = 1, partial: Optional[torch.Tensor] = None) -> None:
    """Causal GQA over the paged cache for any mixture of prompt and decode sequences."""
    if d not in SIMT_HEAD_DIMS:
        raise KernelError(f"attention takes head sizes in steps of 16 up to 512, not {d}")
    _require(q, "q")
    _require(out, "out", q.dtype)
    _require(k_pool, "k_pool", q.dtype)
    _require(v_pool, "v_pool", q.dtype)
    n_tokens = q.numel() // (nq * d)
    if out.numel() != q.numel():
        raise KernelError("q and out disagree")
    if splits > 1:
        need = n_tokens * nq * splits * (d + 2)
        if partial is None or partial.numel() < need or partial.dtype != torch.float32:
            raise KernelError(f"splits={splits} needs an fp32 partial buffer of {need} elements")
    args = _AttnArgs(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), _ptr(partial), _ptr(cu_q), _ptr(past),
                     _ptr(page_start), _ptr(page_ids), n_seqs, nq, nkv, page_size, ring_pages, window, splits,
                     0, 0, scale)
    lib = load_library("attention_simt", {"ODI_HEAD_DIM": d})
    _check(lib.odi_attention_simt(byref(args), c_int(max_q_len), c_int(n_tokens), c_int(dtype_code(q.dtype)),
                                  _stream()), "attention_simt", 2 if splits > 1 else 1)


class _MmaAttnArgs(Structure):
    _fields_ = [("q", c_void_p), ("k_pool", c_void_p), ("v_pool", c_void_p), ("out", c_void_p),
                ("partial", c_void_p), ("cu_q", c_void_p), ("past", c_void_p), ("page_start", c_void_p),
                ("page_ids", c_void_p), ("n_seqs", c_int), ("nq", c_int), ("nkv", c_int), ("splits", c_int),
                ("head_chunks", c_int), ("scale", c_float), ("clustered", c_int), ("tickets", c_void_p),
                ("tiles_per_split", c_void_p), ("pool_rows", c_long), ("status", c_void_p), ("items", c_int),
                ("skip_combine", c_int)]


MMA_HEAD_DIMS = tuple(range(16, 257, 16))

_attention_state = {}


def _attention_tickets(device, count: int) -> torch.Tensor:
    """Counters of the split-key decode attention, one per (sequence, block row); kept zero between launches."""
    have = _attention_state.get(device)
    if have is None or have.numel() < count:
        if have is not None:
            _outgrown.append(have)
        have = torch.zeros(max(count, 4096), dtype=torch.int32, device=device)
        _attention_state[device] = have
    return have


DECODE_ATTENTION_BLOCKS = 296     # blocks of the split-key decode kernel that a B200 holds at once (148 SMs x 2)
ROUND_FILL_CUTS = 6               # the most cuts per sequence when whole sequences already run in rounds


def plan_key_splits(kv_lens: Sequence[int], block_rows: int, *, blocks: int = DECODE_ATTENTION_BLOCKS,
                    min_tiles: int = 2, max_splits: int = 32) -> Tuple[int, int]:
    """How the split-key decode attention cuts unequal sequences: ``(tiles_per_split, splits)``.

    ``kv_lens`` are the keys that each sequence sees, ``block_rows`` the blocks that one split of one
    sequence launches (kv heads x chunks of 16 query heads).  Every block takes ``tiles_per_split`` tiles
    of 64 keys, so a long sequence gets more blocks than a short one and all blocks end together; the
    size is the smallest (from ``min_tiles`` up) with which all blocks are on the GPU at once, or the
    longest sequence whole when even that is too many.  ``splits`` is what the longest sequence needs; more
    than 32 measured slower even where they would fill the GPU exactly (one sequence of 131,072 keys, 8 kv
    heads: 95 us with 32, 103 with 37, 108 with 64), since every split adds to the merge."""
    tiles = [max(1, -(-int(n) // 64)) for n in kv_lens]
    longest, total = max(tiles), sum(tiles)
    per = max(min_tiles, -(-total * block_rows // blocks), -(-longest // max_splits))
    for _ in range(64):
        if per >= longest or sum(-(-t // per) for t in tiles) * block_rows <= blocks:
            break
        per += max(1, per // 8)
    per = min(per, longest)
    if per == longest and len(tiles) * block_rows > blocks:
        # More whole sequences than the GPU holds blocks: they run in rounds, and the last round may be nearly
        # empty (40 sequences x 8 kv heads: 320 blocks on 296 places, two rounds for 1.08).  A few cuts per
        # sequence fill the rounds better.  Estimate: rounds x (tiles of a block + 4 for its start and end), plus
        # 6 for the merge when there are cuts; measured at 2,048 keys (us, whole / best cut): 40 sequences 80 /
        # 69 (3 to 5 cuts), 48: 83 / 76 (3 cuts), 56: 85 / 90, 64: 87 / 101 (whole sequences stay).
        def estimate(size: int) -> float:
            count = sum(-(-t // size) for t in tiles) * block_rows
            return -(-count // blocks) * (size + 4) + (6 if size < longest else 0)
        best, best_cost = longest, estimate(longest)
        for cuts in range(2, min(max_splits, ROUND_FILL_CUTS) + 1):
            size = -(-longest // cuts)
            if size < min_tiles:
                break
            cost = estimate(size)
            if cost < best_cost:
                best, best_cost = size, cost
        per = best
    return per, -(-longest // per)


def key_split_capacity(n_seqs: int, block_rows: int, *, blocks: int = DECODE_ATTENTION_BLOCKS, max_splits: int = 32) -> int:
    """The most (sequence, split) pairs that :func:`plan_key_splits` gives ``n_seqs`` sequences, whatever their
    lengths: what fills the GPU once, or every sequence whole; with more whole sequences than the GPU holds
    blocks, every sequence may be cut ``ROUND_FILL_CUTS`` times."""
    if n_seqs * block_rows > blocks:
        return n_seqs * min(max_splits, ROUND_FILL_CUTS)
    return min(n_seqs * max_splits, max(n_seqs, blocks // block_rows))


def key_split_list(kv_lens: Sequence[int], tiles_per_split: int, capacity: int) -> List[int]:
    """The decode attention's list of blocks for sequences of ``kv_lens`` keys cut every ``tiles_per_split`` tiles
    of 64: ``[tiles_per_split, n, entry...]`` padded with zeros to ``2 + capacity``.  An entry is
    ``sequence << 8 | 128 if it is the sequence's last | split``; blocks with the most tiles come first, so that
    when the blocks run in more than one round the short ones fill the end.  The list holds for every bound on
    the splits that the longest sequence fits (``splits * tiles_per_split`` tiles)."""
    per = max(1, int(tiles_per_split))
    entries = []
    for seq, n in enumerate(kv_lens):
        tiles = max(1, -(-int(n) // 64))
        count = -(-tiles // per)
        if count > 128:
            raise KernelError(f"{count} blocks for one sequence; an entry of the list holds up to 128")
        entries.extend((-per, seq, split, False) for split in range(count - 1))
        entries.append((-(tiles - (count - 1) * per), seq, count - 1, True))
    if len(entries) > capacity:
        raise KernelError(f"{len(entries)} blocks of keys for a list of {capacity}: the plan and the graph disagree")
    entries.sort()
    packed = [(seq << 8) | (128 if last else 0) | split for _, seq, split, last in entries]
    return [per, len(packed)] + packed + [0] * (capacity - len(packed))


def attention_mma(q, k_pool, v_pool, out, cu_q, past, page_start, page_ids, *, n_seqs: int, max_q_len: int,
                  nq: int, nkv: int, d: int, page_size: int, scale: float, splits: int = 1,
                  partial: Optional[torch.Tensor] = None, cluster: bool = False, merge_in_kernel: bool = False,
                  tiles_per_split: Optional[torch.Tensor] = None, combine: bool = True) -> None:
    """bf16 causal GQA on the tensor cores: the prefill kernel for any q_len, the split-key
    decode kernel when every sequence brings exactly one token.  No window.

    Decode with ``tiles_per_split`` (int32 on the device, written by the host; see
    :func:`plan_key_splits`): every block takes that many tiles of 64 keys and ``splits`` only bounds the
    count per sequence; whatever the number says, ``splits`` blocks cover every sequence.  With one element the
    grid has ``splits`` blocks for every sequence and those without keys leave at once; with more it is a
    :func:`key_split_list`, the grid is as long as the list's capacity (or ``n_seqs * splits`` if that is less),
    and a list that does not cover the lengths on the device is reported through the kernels' status word.  Without it every sequence is cut into
    ``splits`` equal ranges.

    Decode splits go through the fp32 ``partial`` buffer and a combine kernel; ``combine=False`` leaves them in
    ``partial`` unmerged (``out`` may then be None) for a product that takes them as its operand
    (:func:`gemm_bf16` with ``merge``).  ``merge_in_kernel=True``
    lets the block that finishes a (sequence, kv head) last merge them instead (an atomic ticket; the same
    bits); on B200 that measured slower (20.1 against 17.5 us at 8 x 2048 with 4 splits, 17.1 against 10.8 us
    at 1 x 2048 with 16: the fence, the ticket and the merge lengthen the slowest block).  ``cluster=True``
    merges 2..8 splits inside a thread-block cluster instead (no scratch, no second kernel); on
    B200 that measured no faster (19.4 against 19.3 us at 8 x 2048, slower at other split counts:
    the co-scheduling of 104 KB blocks costs what the saved launch gains), so it is not the default."""
    if d not in MMA_HEAD_DIMS:
        raise KernelError(f"the tensor-core attention takes head sizes in steps of 16 up to 256, not {d}")
    if page_size != 64:
        raise KernelError("the tensor-core attention works on pages of 64 positions")
    _require(q, "q", torch.bfloat16)
    _require(k_pool, "k_pool", torch.bfloat16)
    _require(v_pool, "v_pool", torch.bfloat16)
    n_tokens = q.numel() // (nq * d)
    decode = max_q_len == 1
    if not decode:
        splits = 1
    clustered = cluster and 1 < splits <= 8
    if not combine and (not decode or splits == 1 or clustered or merge_in_kernel):
        raise KernelError("combine=False belongs to the decode kernel with more than one split and global partials")
    if combine or out is not None:
        _require(out, "out", torch.bfloat16)
        if out.numel() != q.numel():
            raise KernelError("q and out disagree")
    if splits > 1 and not clustered:
        need = n_tokens * nq * splits * (d + 2)
        if partial is None or partial.numel() < need or partial.dtype != torch.float32:
            raise KernelError(f"splits={splits} needs an fp32 partial buffer of {need} elements")
    tickets = None
    if decode and splits > 1 and not clustered and merge_in_kernel:
        tickets = _attention_tickets(q.device, n_seqs * nkv * (-(-(nq // nkv) // 16)))
    if tiles_per_split is not None:
        if not decode or clustered or tickets is not None:
            raise KernelError("tiles_per_split belongs to the decode kernel with the combine kernel")
        _require(tiles_per_split, "tiles_per_split", torch.int32)
        if tiles_per_split.numel() == 2:
            raise KernelError("tiles_per_split is one number or a list of 2 + capacity")
    # the grid: as long as the list, but no longer than `splits` blocks for every sequence, which no list exceeds
    # (blocks behind the list's end leave at once, yet each costs a place on an SM for a moment: 64 whole
    # sequences on a grid for six cuts each measured 4 % more per step)
    items = min(tiles_per_split.numel() - 2, n_seqs * splits) if tiles_per_split is not None and tiles_per_split.numel() > 1 else 0
    # what the TMA-fed decode form needs besides: the pools' extent (rows of d) and the error word of its bounded waits
    pool_rows = k_pool.numel() // d if k_pool.numel() == v_pool.numel() else 0
    _, _, status = _gemm_buffers(q.device, 0)
    args = _MmaAttnArgs(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), _ptr(partial), _ptr(cu_q), _ptr(past),
                        _ptr(page_start), _ptr(page_ids), n_seqs, nq, nkv, splits, 0, scale, 1 if clustered else 0,
                        _ptr(tickets), _ptr(tiles_per_split if decode else None), pool_rows, _ptr(status), items,
                        0 if combine else 1)
    lib = load_library("attention_mma", {"ODI_HEAD_DIM": d})
    _check(lib.odi_attention_mma(byref(args), c_int(max_q_len), c_int(n_tokens), c_int(1 if decode else 0),
                                 _stream()), "attention_mma",
           2 if (splits > 1 and not clustered and tickets is None and combine) else 1)


def attention_mma_combine(partial: torch.Tensor, out: torch.Tensor, past: torch.Tensor, *, nq: int, d: int, splits: int,
                          tiles_per_split: Optional[torch.Tensor] = None) -> None:
    """Merge the ``splits`` partials per token and head that :func:`attention_mma` left with ``combine=False``
    into ``out`` [tokens, nq * d] (the kernel that the launch would have run itself)."""
    _require(partial, "partial", torch.float32)
    _require(out, "out", torch.bfloat16)
    _require(past, "past", torch.int32, 1)
    tokens = past.numel()
    if d not in MMA_HEAD_DIMS or out.numel() != tokens * nq * d or partial.numel() < tokens * nq * splits * (d + 2):
        raise KernelError("attention_mma_combine: sizes disagree")
    if tiles_per_split is not None:
        _require(tiles_per_split, "tiles_per_split", torch.int32)
    lib = load_library("attention_mma", {"ODI_HEAD_DIM": d})
    _check(lib.odi_attention_mma_combine(_ptr(partial), _ptr(out), c_int(tokens), c_int(nq), c_int(splits), _ptr(past),
                                         _ptr(tiles_per_split), _stream()), "attention_mma_combine")


class _TcAttnArgs(Structure):
    _fields_ = [("out", c_void_p), ("cu_q", c_void_p), ("past", c_void_p), ("page_start", c_void_p),
                ("page_ids", c_void_p), ("status", c_void_p), ("n_seqs", c_int), ("nq", c_int), ("nkv", c_int),
                ("scale", c_float)]


TCGEN05_ATTENTION_HEAD_DIMS = (64, 128)


def attention_tcgen05(q, k_pool, v_pool, out, cu_q, past, page_start, page_ids, *, n_seqs: int, max_q_len: int,
                      nq: int, nkv: int, d: int, page_size: int, scale: float, heads_per_cta: int = 0) -> None:
    """bf16 causal GQA for prefill on tcgen05: scores and outputs in tensor memory, TMA-fed pages.
    ``heads_per_cta``: 1, or 2 (two heads of a key/value group share a CTA and its K/V pages; needs an
    even group size), or 0 for the library's choice."""
    if d not in TCGEN05_ATTENTION_HEAD_DIMS:
        raise KernelError(f"the tcgen05 attention takes head sizes {TCGEN05_ATTENTION_HEAD_DIMS}, not {d}")
    if page_size != 64:
        raise KernelError("the tcgen05 attention works on pages of 64 positions")
    for name, t in (("q", q), ("out", out), ("k_pool", k_pool), ("v_pool", v_pool)):
        _require(t, name, torch.bfloat16)
    n_tokens = q.numel() // (nq * d)
    if out.numel() != q.numel() or k_pool.shape != v_pool.shape or k_pool.dim() != 4:
        raise KernelError("attention_tcgen05: q/out or the pools disagree")
    _, _, status = _gemm_buffers(q.device, 0)
    args = _TcAttnArgs(_ptr(out), _ptr(cu_q), _ptr(past), _ptr(page_start), _ptr(page_ids), _ptr(status),
                       n_seqs, nq, nkv, scale)
    lib = load_library("attention_tcgen05", {"ODI_HEAD_DIM": d})
    _check(lib.odi_attention_tcgen05(_ptr(q), _ptr(k_pool), _ptr(v_pool), byref(args), c_int(n_tokens),
                                     c_int(max_q_len), c_long(k_pool.shape[0]), c_int(heads_per_cta), _stream()),
           "attention_tcgen05")


# ------------------------------------------------------------------------------ sampling


_sample_state = {}


def _sample_buffers(device, rows: int, chunks: int):
    """Per-chunk partial results (16 bytes each) and one ticket per row (kept zero between launches)."""
    state = _sample_state.setdefault(device, {})
    if state.get("rows", 0) < rows:
        _outgrown.append(state.get("tickets"))
        state["tickets"] = torch.zeros(max(rows, 256), dtype=torch.int32, device=device)
        state["rows"] = state["tickets"].numel()
    if state.get("entries", 0) < rows * chunks:
        _outgrown.append(state.get("partials"))
        state["partials"] = torch.empty(max(rows * chunks, 4096) * 4, dtype=torch.float32, device=device)
        state["entries"] = state["partials"].numel() // 4
    return state["partials"], state["tickets"]


def sample(logits: torch.Tensor, out: torch.Tensor, temperature: float, seed: int = 0,
           streams: Optional[torch.Tensor] = None, steps: Optional[torch.Tensor] = None, *,
           advance_pos: Optional[torch.Tensor] = None, advance_past: Optional[torch.Tensor] = None,
           active: Optional[torch.Tensor] = None) -> None:
    """out[i] = argmax(logits[i]) if temperature == 0 else a draw from softmax(logits[i] / temperature).

    With ``active`` (int32 0/1 per row) the kernel also adds ``active[i]`` to ``advance_pos[i]``,
    ``advance_past[i]`` and ``steps[i]``: the bookkeeping of a decode loop that stays on the device."""
    _require(logits, "logits", torch.float32, 2)
    _require(out, "out", torch.int32, 1)
    n, V = logits.shape
    if out.numel() < n:
        raise KernelError("out is shorter than the number of rows")
    if temperature > 0:
        _require(streams, "streams", torch.int32, 1)
        _require(steps, "steps", torch.int32, 1)
    if active is not None:
        for name, t in (("active", active), ("advance_pos", advance_pos), ("advance_past", advance_past)):
            _require(t, name, torch.int32, 1)
    lib = load_library("sampling")
    partials, tickets = _sample_buffers(logits.device, n, int(lib.odi_sample_chunks(c_int(V))))
    _check(lib.odi_sample(_ptr(logits), _ptr(out), c_int(n), c_int(V), c_int(V), c_float(temperature),
                          c_ulonglong(seed & ((1 << 64) - 1)), _ptr(streams), _ptr(steps), _ptr(advance_pos),
                          _ptr(advance_past), _ptr(active), _ptr(partials), _ptr(tickets), _stream()), "sample")
