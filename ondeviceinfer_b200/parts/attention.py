"""Grouped-query causal attention over the paged cache
(ondeviceinfer/attention.py:88-177 of UESlubei/ondeviceinfer).

Steps of ``forward``: one matrix product for the concatenated q, k, v projections (with their
biases, if the spec names any: ondeviceinfer/attention.py:106-123); the
per-head Q/K RMSNorm, the rotary embedding and the cache write (a fused kernel of their own,
or, at decode widths with heads of 128, the epilogue of that product); attention over the
cache pages of each sequence; the output projection with the residual add.  Head counts,
head size, eps, window, scale and the position encoding are all fields of the spec.
"""

from __future__ import annotations

import math

import torch

from ..cache import PAGE_SIZE, KVNeed
from ..config.specs import AttentionSpec
from ..kernels import ops
from ..weights.tensors import TensorDecl
from .base import Part, build_part, register_part
from .linear import UnmergedSplits, heads_in_epilogue, linear, merge_in_product, project_heads


TCGEN05_MIN_Q_LEN = 16     # shorter chunks fill too little of a 128-row tile


class Attention(Part):
    graph_safe = True   # no host work that depends on the step's values: may be captured in a CUDA graph
    takes_lazy_norm = True   # x may be a NormedRows: its first product makes the normed operand itself

    def __init__(self, spec: AttentionSpec) -> None:
        super().__init__(spec)
        if spec.num_heads % spec.num_kv_heads != 0:
            raise ValueError("Q heads must be divisible by KV heads for GQA")
        if spec.head_dim % 16 != 0 or not 16 <= spec.head_dim <= 512:
            raise ValueError(f"head_dim={spec.head_dim}: the attention kernels take multiples of 16 up to 512")
        if spec.window is not None and spec.window <= 0:
            raise ValueError("window must be positive")
        self.position = build_part(spec.position)
        self.scale = spec.scale if spec.scale is not None else 1.0 / math.sqrt(spec.head_dim)

    # ------------------------------------------------------------------ tensors

    def tensor_decls(self):
        s = self.spec
        q, kv = s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim
        decls = [TensorDecl(s.name("q"), (q, s.hidden_size)), TensorDecl(s.name("k"), (kv, s.hidden_size)),
                 TensorDecl(s.name("v"), (kv, s.hidden_size)), TensorDecl(s.name("o"), (s.hidden_size, q))]
        if s.qk_norm_eps is not None:
            decls += [TensorDecl(s.name("q_norm"), (s.head_dim,), "one_plus_normal"),
                      TensorDecl(s.name("k_norm"), (s.head_dim,), "one_plus_normal")]
        decls += [TensorDecl(s.name(role), (size,)) for role, size in
                  (("q_bias", q), ("k_bias", kv), ("v_bias", kv), ("o_bias", s.hidden_size)) if s.has(role)]
        return decls + self.position.tensor_decls()

    def load(self, fetch, runtime) -> None:
        s = self.spec
        self.runtime = runtime
        # q, k and v rows concatenated: one product yields [tokens, (nq + 2 nkv) * d]
        self.w_qkv = torch.cat([fetch.matrix(s.name("q")), fetch.matrix(s.name("k")), fetch.matrix(s.name("v"))], 0)
        self.w_o = fetch.matrix(s.name("o"))
        self.q_norm = fetch.vector(s.name("q_norm")) if s.qk_norm_eps is not None else None
        self.k_norm = fetch.vector(s.name("k_norm")) if s.qk_norm_eps is not None else None
        # biases (fp32), those of q, k and v concatenated like their weights; a projection without one adds zero
        q, kv = s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim
        self.b_qkv = None
        if any(s.has(role) for role in ("q_bias", "k_bias", "v_bias")):
            zeros = lambda size: torch.zeros(size, dtype=torch.float32, device=runtime.device)
            self.b_qkv = torch.cat([fetch.vector(s.name(role)) if s.has(role) else zeros(size)
                                    for role, size in (("q_bias", q), ("k_bias", kv), ("v_bias", kv))])
        self.b_o = fetch.vector(s.name("o_bias")) if s.has("o_bias") else None
        self.position.load(fetch, runtime)

    def cache_needs(self):
        return (KVNeed(self.spec.num_kv_heads, self.spec.head_dim, self.spec.window),)

    # ------------------------------------------------------------------ step

    def forward(self, x, ctx, view, residual) -> None:
        s = self.spec
        n = x.shape[0]
        group = view.kv_group
        page_start, page_ids = ctx.page_table(group.index)
        q = torch.empty((n, s.num_heads * s.head_dim), dtype=x.dtype, device=x.device)
        tables = self.position.rotary_tables(ctx)
        cos, sin = tables if tables is not None else (None, None)
        # with heads of 128 at decode widths the product's epilogue prepares the heads itself
        fused = heads_in_epilogue(x, self.w_qkv, head_dim=s.head_dim, rot_dim=self.position.rot_dim,
                                  rotated=cos is not None, write_kv=view.writes_kv, biased=self.b_qkv is not None)
        prepared = ops.head_prep(None if fused else linear(x, self.w_qkv, bias=self.b_qkv), q, view.keys, view.values,
                                 self.q_norm, self.k_norm, cos, sin, ctx.tok_seq, ctx.tok_pos, page_start, page_ids,
                                 nq=s.num_heads, nkv=s.num_kv_heads, d=s.head_dim, rot_dim=self.position.rot_dim,
                                 page_size=PAGE_SIZE, ring_pages=group.ring_pages, write_kv=view.writes_kv,
                                 eps=s.qk_norm_eps if s.qk_norm_eps is not None else 0.0)
        if fused:
            project_heads(x, self.w_qkv, prepared, bias=self.b_qkv)
        o = self.attend(q, ctx, view, page_start, page_ids)
        linear(o, self.w_o, bias=self.b_o, residual=residual, track=ctx)

    def attend(self, q, ctx, view, page_start, page_ids):
        """The attention output [tokens, heads * head size], or, from a decode step whose key splits the output
        projection can merge itself, those splits unmerged (:class:`~ondeviceinfer_b200.parts.linear.UnmergedSplits`).

        bf16 without a window: the tensor-core kernels -- tcgen05 flash attention for steps that
        bring more than 16 tokens per sequence (head sizes 64 and 128), the mma.sync prefill form for
        short chunks and other head sizes, the split-key decode form when every sequence brings one
        token.  float32, windows, head sizes above 256: the CUDA-core kernel."""
        s = self.spec
        tensor_cores = q.dtype == torch.bfloat16 and s.window is None and s.head_dim <= 256
        splits, partial, tiles_per_split = 1, None, None
        if ctx.max_q_len == 1:
            # decode: cut long key ranges so that enough blocks run side by side
            block_rows = s.num_kv_heads * ((s.num_heads // s.num_kv_heads + 15) // 16)
            if tensor_cores:
                # blocks of equal size, so that unequal sequences end together; the context plans it
                tiles_per_split, splits = ctx.key_splits(block_rows)
            else:
                splits = max(1, min(32, 296 // max(ctx.n_seqs * block_rows, 1), (ctx.max_kv_len + 255) // 256))
            if splits > 1:
                partial = torch.empty((ctx.n_tokens * s.num_heads * splits * (s.head_dim + 2),),
                                      dtype=torch.float32, device=q.device)
        if tensor_cores and ctx.max_q_len == 1 and splits > 1 and merge_in_product(
                ctx.n_tokens, self.w_o, splits=splits, heads=s.num_heads, head_dim=s.head_dim, biased=self.b_o is not None):
            # the output projection merges the splits in its prologue: no combine kernel, no bf16 round trip
            ops.attention_mma(q, view.keys, view.values, None, ctx.cu_q, ctx.past, page_start, page_ids,
                              n_seqs=ctx.n_seqs, max_q_len=1, nq=s.num_heads, nkv=s.num_kv_heads, d=s.head_dim,
                              page_size=PAGE_SIZE, scale=self.scale, splits=splits, partial=partial,
                              tiles_per_split=tiles_per_split, combine=False)
            return UnmergedSplits(partial, ctx.past, tiles_per_split, splits=splits, heads=s.num_heads,
                                  head_dim=s.head_dim)
        o = torch.empty_like(q)
        if tensor_cores and ctx.max_q_len > TCGEN05_MIN_Q_LEN and s.head_dim in ops.TCGEN05_ATTENTION_HEAD_DIMS:
            ops.attention_tcgen05(q, view.keys, view.values, o, ctx.cu_q, ctx.past, page_start, page_ids,
                                  n_seqs=ctx.n_seqs, max_q_len=ctx.max_q_len, nq=s.num_heads, nkv=s.num_kv_heads,
                                  d=s.head_dim, page_size=PAGE_SIZE, scale=self.scale)
            return o
        if tensor_cores:
            ops.attention_mma(q, view.keys, view.values, o, ctx.cu_q, ctx.past, page_start, page_ids,
                              n_seqs=ctx.n_seqs, max_q_len=ctx.max_q_len, nq=s.num_heads, nkv=s.num_kv_heads,
                              d=s.head_dim, page_size=PAGE_SIZE, scale=self.scale, splits=splits, partial=partial,
                              tiles_per_split=tiles_per_split if ctx.max_q_len == 1 else None)
            return o
        ops.attention_simt(q, view.keys, view.values, o, ctx.cu_q, ctx.past, page_start, page_ids,
                           n_seqs=ctx.n_seqs, max_q_len=ctx.max_q_len, nq=s.num_heads, nkv=s.num_kv_heads,
                           d=s.head_dim, page_size=PAGE_SIZE, ring_pages=view.kv_group.ring_pages,
                           window=s.window or 0, scale=self.scale, splits=splits, partial=partial)
        return o


register_part(AttentionSpec, Attention)
