"""Timing single kernels at given sizes: ``python -m ondeviceinfer_b200.kernels.microbench <case> ...``

Each case runs one kernel of the library on synthetic data with CUDA-event timing after
warm-up.  Operands that a decode step reads once (weights, cached keys and values) are
rotated over several copies larger than the 126 MB L2 together, so that the figures are
HBM figures.  The same command line is what the ``ncu`` summaries under ``profiles/`` were
captured with (on small cases).

Cases: ``gemm`` (tcgen05 GEMM, or the library's with ``--library``), ``attention-decode``,
``attention-prefill``, ``rmsnorm``, ``sample``.
"""

from __future__ import annotations

import argparse
import json
import math

import torch

from . import ops

L2_BYTES = 126e6


def time_kernel(run, variants: int, reps: int, warmup: int = 3) -> float:
    """Mean microseconds of ``run(i)`` cycling i over ``variants`` operand sets.

    The launches are captured into one CUDA graph and the graph is replayed, so the figure
    is device time per kernel as in a captured decode step (consecutive kernels overlap their
    launch and set-up through programmatic dependent launch), not host launch throughput."""
    for i in range(max(warmup, 1)):
        run(i % variants)
    torch.cuda.synchronize()
    per_graph = max(variants, 8)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        run(0)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(per_graph):
            run(i % variants)
    graph.replay()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(reps):
        graph.replay()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) * 1000.0 / (reps * per_graph)


def gemm_case(args) -> dict:
    epi = {"store_bf16": ops.EPI_STORE_BF16, "store_f32": ops.EPI_STORE_F32, "residual": ops.EPI_RESIDUAL,
           "swiglu": ops.EPI_SWIGLU, "head_prep": ops.EPI_HEAD_PREP}[args.epi]
    rows = 2 * args.n if epi == ops.EPI_SWIGLU else args.n
    copies = max(1, int(math.ceil(3 * L2_BYTES / (rows * args.k * 2)))) if args.rotate else 1
    ws = [(torch.randn(rows, args.k, device="cuda") / math.sqrt(args.k)).bfloat16() for _ in range(copies)]
    x = torch.randn(args.tokens, args.k, device="cuda").bfloat16()
    wide = epi in (ops.EPI_STORE_F32, ops.EPI_RESIDUAL)
    out = torch.zeros(args.tokens, args.n, dtype=torch.float32 if wide else torch.bfloat16, device="cuda")
    extra = {}
    if args.norm:      # the operand comes through the fused RMSNorm: fp32 rows and their sums of squares
        hidden = torch.randn(args.tokens, args.k, device="cuda")
        parts = torch.zeros(ops.gemm_bf16_sumsq_parts(args.k), args.tokens, device="cuda")
        padded = torch.zeros(args.tokens, parts.shape[0] * 128, device="cuda")
        padded[:, :args.k] = hidden
        parts.copy_((padded.view(args.tokens, -1, 128) ** 2).sum(-1).t())
        extra["norm"] = (hidden, torch.ones(args.k, device="cuda"), parts, 1e-6)
        x = None
    if epi == ops.EPI_RESIDUAL and args.sumsq:
        extra["sumsq_out"] = torch.empty(ops.gemm_bf16_sumsq_parts(args.n), args.tokens, device="cuda")
    if epi == ops.EPI_HEAD_PREP:   # rows of w are query, key and value heads of 128 (4 query heads per kv head)
        d, heads = 128, args.n // 128
        nkv = heads // 6
        nq = heads - 2 * nkv
        pools, page_start, page_ids = _cache_setup(args.tokens, args.ctx, nkv, d, 1)
        tok = torch.arange(args.tokens, dtype=torch.int32, device="cuda")
        pos = torch.full((args.tokens,), args.ctx - 1, dtype=torch.int32, device="cuda")
        cos = torch.ones(args.tokens, d // 2, device="cuda")
        sin = torch.zeros(args.tokens, d // 2, device="cuda")
        ones = torch.ones(d, device="cuda")
        q_out = torch.empty(args.tokens, nq * d, dtype=torch.bfloat16, device="cuda")
        extra["head_prep"] = ops.head_prep(None, q_out, pools[0][0], pools[0][1], ones, ones, cos, sin, tok, pos,
                                           page_start, page_ids, nq=nq, nkv=nkv, d=d, rot_dim=d, page_size=64,
                                           ring_pages=0, write_kv=True, eps=1e-6)
        out = None
    if args.library:
        run = lambda i: torch.matmul(x, ws[i].t())
    elif args.persistent:
        run = lambda i: ops.gemm_prefill_bf16(x, ws[i], out, epi)
    else:
        run = lambda i: ops.gemm_bf16(x, ws[i], out, epi, bn=args.bn, splits=args.splits,
                                      cluster=not args.no_cluster, **extra)
    us = time_kernel(run, copies, args.reps)
    ops.raise_on_kernel_fault()
    weight_bytes, flops = rows * args.k * 2, 2.0 * args.tokens * rows * args.k
    return {"case": "gemm", "tokens": args.tokens, "n": args.n, "k": args.k, "epi": args.epi, "norm": bool(args.norm),
            "plan": None if args.library else list(ops.gemm_bf16_plan(args.tokens, args.n, args.k, epi)),
            "us": us, "weight_GBps": weight_bytes / us / 1e3, "TFLOPs": flops / us / 1e6}


def _cache_setup(batch: int, ctx: int, nkv: int, d: int, copies: int, in_order: bool = False):
    pages_per_seq = (ctx + 64) // 64 + 1
    n_pages = batch * pages_per_seq
    pools = [torch.randn(2, n_pages, nkv, 64, d, device="cuda").bfloat16() for _ in range(copies)]
    order = (torch.arange(n_pages) if in_order else torch.randperm(n_pages)).to(torch.int32)
    page_ids = order.cuda()
    page_start = (torch.arange(batch + 1, dtype=torch.int32) * pages_per_seq).cuda()
    return pools, page_start, page_ids


def _decode_lengths(args) -> list:
    """``--lengths``: ``a,b,c`` (one sequence each) or ``LO-HI@SEED`` (``--batch`` random lengths); default ``--ctx`` each."""
    if not args.lengths:
        return [args.ctx] * args.batch
    if "@" in args.lengths:
        span, seed = args.lengths.split("@")
        lo, hi = (int(v) for v in span.split("-"))
        return torch.randint(lo, hi + 1, (args.batch,), generator=torch.Generator().manual_seed(int(seed))).tolist()
    return [int(v) for v in args.lengths.split(",")]


def attention_decode_case(args) -> dict:
    nq, nkv, d = args.heads, args.kv_heads, args.head_dim
    lengths = _decode_lengths(args)
    batch = len(lengths)
    kv_bytes = 2 * sum(lengths) * nkv * d * 2
    copies = max(1, int(math.ceil(3 * L2_BYTES / kv_bytes))) if args.rotate else 1
    pools, page_start, page_ids = _cache_setup(batch, max(lengths), nkv, d, copies, args.pages_in_order)
    q = torch.randn(batch, nq, d, device="cuda").bfloat16()
    out = torch.empty(batch, nq * d, dtype=torch.bfloat16, device="cuda")
    cu_q = torch.arange(batch + 1, dtype=torch.int32, device="cuda")
    past = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device="cuda")
    splits, blocks, plan = args.splits, None, None
    if args.planned:       # as a decode step does it: blocks of equal size from the plan, listed by the host
        block_rows = nkv * -(-(nq // nkv) // 16)
        per, needed = ops.plan_key_splits(lengths, block_rows)
        splits = 1
        while splits < needed:
            splits *= 2
        blocks = torch.tensor(ops.key_split_list(lengths, per, ops.key_split_capacity(batch, block_rows)),
                              dtype=torch.int32, device="cuda")
        plan = {"tiles_per_split": per, "splits": needed, "bound": splits, "blocks": int(blocks[1]) * block_rows}
    partial = torch.empty(batch * nq * splits * (d + 2), dtype=torch.float32, device="cuda") if splits > 1 else None
    run = lambda i: ops.attention_mma(q, pools[i][0], pools[i][1], out, cu_q, past, page_start, page_ids,
                                      n_seqs=batch, max_q_len=1, nq=nq, nkv=nkv, d=d, page_size=64,
                                      scale=1 / math.sqrt(d), splits=splits, partial=partial, tiles_per_split=blocks,
                                      cluster=args.cluster_attention, merge_in_kernel=args.merge_in_kernel)
    us = time_kernel(run, copies, args.reps)
    ops.raise_on_kernel_fault()
    return {"case": "attention-decode", "batch": batch, "keys": sum(lengths), "longest": max(lengths), "splits": splits,
            "plan": plan, "us": us, "kv_GBps": kv_bytes / us / 1e3}


def attention_prefill_case(args) -> dict:
    nq, nkv, d, T = args.heads, args.kv_heads, args.head_dim, args.tokens
    pools, page_start, page_ids = _cache_setup(args.batch, T, nkv, d, 1)
    q = torch.randn(args.batch * T, nq, d, device="cuda").bfloat16()
    out = torch.empty(args.batch * T, nq * d, dtype=torch.bfloat16, device="cuda")
    cu_q = (torch.arange(args.batch + 1, dtype=torch.int32) * T).cuda()
    past = torch.zeros(args.batch, dtype=torch.int32, device="cuda")
    extra = {} if args.mma_sync else {"heads_per_cta": args.heads_per_cta}
    kernel = ops.attention_mma if args.mma_sync else ops.attention_tcgen05
    run = lambda i: kernel(q, pools[0][0], pools[0][1], out, cu_q, past, page_start, page_ids, n_seqs=args.batch,
                           max_q_len=T, nq=nq, nkv=nkv, d=d, page_size=64, scale=1 / math.sqrt(d), **extra)
    us = time_kernel(run, 1, args.reps)
    ops.raise_on_kernel_fault()
    flops = 2.0 * args.batch * nq * d * T * T          # causal half of 4 * T^2 * d per head
    return {"case": "attention-prefill", "batch": args.batch, "tokens": T, "us": us, "TFLOPs": flops / us / 1e6}


def rmsnorm_case(args) -> dict:
    x = torch.randn(args.tokens, args.n, device="cuda")
    w = torch.ones(args.n, device="cuda")
    out = torch.empty(args.tokens, args.n, dtype=torch.bfloat16, device="cuda")
    us = time_kernel(lambda i: ops.rmsnorm(x, w, 1e-6, out), 1, args.reps)
    return {"case": "rmsnorm", "tokens": args.tokens, "n": args.n, "us": us,
            "GBps": args.tokens * args.n * 6 / us / 1e3}


def sample_case(args) -> dict:
    logits = torch.randn(args.tokens, args.n, device="cuda")
    out = torch.empty(args.tokens, dtype=torch.int32, device="cuda")
    streams = torch.arange(args.tokens, dtype=torch.int32, device="cuda")
    steps = torch.zeros(args.tokens, dtype=torch.int32, device="cuda")
    us = time_kernel(lambda i: ops.sample(logits, out, args.temperature, 1, streams, steps), 1, args.reps)
    return {"case": "sample", "rows": args.tokens, "vocab": args.n, "temperature": args.temperature, "us": us}


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="python -m ondeviceinfer_b200.kernels.microbench", description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("case", choices=("gemm", "attention-decode", "attention-prefill", "rmsnorm", "sample"))
    parser.add_argument("--tokens", type=int, default=8)
    parser.add_argument("--n", type=int, default=4096)
    parser.add_argument("--k", type=int, default=4096)
    parser.add_argument("--epi", default="store_bf16", choices=("store_bf16", "store_f32", "residual", "swiglu", "head_prep"))
    parser.add_argument("--norm", action="store_true", help="gemm: the operand through the fused RMSNorm prologue")
    parser.add_argument("--sumsq", action="store_true", help="gemm --epi residual: also leave the rows' sums of squares")
    parser.add_argument("--bn", type=int, default=None)
    parser.add_argument("--splits", type=int, default=None)
    parser.add_argument("--library", action="store_true", help="time the vendor library's product instead")
    parser.add_argument("--persistent", action="store_true", help="gemm: the persistent two-CTA kernel for many tokens")
    parser.add_argument("--no-cluster", action="store_true", help="GEMM K splits through global scratch, not a cluster")
    parser.add_argument("--cluster-attention", action="store_true", help="merge decode-attention splits inside a cluster")
    parser.add_argument("--merge-in-kernel", action="store_true",
                        help="decode-attention splits merged by the block that comes last, not by a second kernel")
    parser.add_argument("--mma-sync", action="store_true", help="attention-prefill: the mma.sync kernel instead of tcgen05")
    parser.add_argument("--heads-per-cta", type=int, default=0, help="attention-prefill on tcgen05: 1, 2 or 0 (default choice)")
    parser.add_argument("--pages-in-order", action="store_true",
                        help="attention-decode: every sequence's pages lie one after another in the pool, as a fresh cache hands them out")
    parser.add_argument("--lengths", default="", help="attention-decode: a,b,c or LO-HI@SEED for --batch random lengths")
    parser.add_argument("--planned", action="store_true",
                        help="attention-decode: the cut that a decode step plans for these lengths, not --splits equal ranges")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--ctx", type=int, default=2048)
    parser.add_argument("--heads", type=int, default=32)
    parser.add_argument("--kv-heads", type=int, default=8)
    parser.add_argument("--head-dim", type=int, default=128)
    parser.add_argument("--temperature", type=float, default=0.0)
    parser.add_argument("--reps", type=int, default=5)
    parser.add_argument("--no-rotate", dest="rotate", action="store_false",
                        help="one operand set only (small captures under a profiler)")
    args = parser.parse_args(argv)
    if args.case == "attention-decode" and args.splits is None:
        args.splits = 1
    torch.manual_seed(0)
    result = {"gemm": gemm_case, "attention-decode": attention_decode_case,
              "attention-prefill": attention_prefill_case, "rmsnorm": rmsnorm_case, "sample": sample_case}[args.case](args)
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
