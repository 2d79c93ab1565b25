"""Host side of the step function: what is wanted, what is refused, the step's index tensors (no GPU)."""

import pytest
import torch

from ondeviceinfer_b200.cache import PAGE_SIZE, KVNeed, SequenceCache
from ondeviceinfer_b200.engine.step import StepContext, resolve_want, validate_step


def make_cache(**kw):
    return SequenceCache([(KVNeed(1, 16),), (KVNeed(1, 16, window=8),)], [None, None], dtype=torch.float32,
                         device="cpu", max_tokens=16 * PAGE_SIZE, max_seqs=4, max_step_tokens=64, **kw)


def test_resolve_want():
    assert resolve_want("last", [3, 1]) == [[2], [0]]
    assert resolve_want("all", [2, 1]) == [[0, 1], [0]]
    assert resolve_want("none", [2, 1]) == [[], []]
    assert resolve_want([[0, 2], []], [3, 1]) == [[0, 2], []]
    with pytest.raises(ValueError):
        resolve_want([[3]], [3])
    with pytest.raises(ValueError):
        resolve_want([[0]], [3, 1])
    with pytest.raises(ValueError):
        resolve_want("first", [1])


def test_validate_step():
    cache = make_cache()
    a, b = cache.alloc(), cache.alloc()
    validate_step(cache, [a, b], [[1, 2], [3]], 10)
    for slots, tokens in (([a], [[1], [2]]), ([], []), ([a, a], [[1], [2]]), ([a], [[]]), ([3], [[1]]),
                          ([a], [[10]]), ([a], [[-1]])):
        with pytest.raises(ValueError):
            validate_step(cache, slots, tokens, 10)


def test_step_context_indexes_tokens_by_sequence_and_position():
    cache = make_cache()
    a, b, c = cache.alloc(), cache.alloc(), cache.alloc()
    cache.reserve([b], [70])
    cache.advance([b], [70])
    tokens = [[5, 6, 7], [8], [9, 10]]
    cache.reserve([a, b, c], [3, 1, 2])
    ctx = StepContext(cache, [a, b, c], tokens, [2, 3, 5], "cpu")
    assert (ctx.n_seqs, ctx.n_tokens, ctx.max_q_len, ctx.max_kv_len, ctx.n_want) == (3, 6, 3, 71, 3)
    assert ctx.token_ids.tolist() == [5, 6, 7, 8, 9, 10]
    assert ctx.tok_seq.tolist() == [0, 0, 0, 1, 2, 2]
    assert ctx.tok_pos.tolist() == [0, 1, 2, 70, 0, 1]
    assert ctx.cu_q.tolist() == [0, 3, 4, 6]
    assert ctx.past.tolist() == [0, 70, 0]
    assert ctx.slots.tolist() == [a, b, c]
    assert ctx.want_rows.tolist() == [2, 3, 5]
    for g, group in enumerate(cache.kv_groups):
        start, ids = ctx.page_table(g)
        assert start.tolist() == [0, len(group.slot_pages[a]), len(group.slot_pages[a]) + len(group.slot_pages[b]),
                                  sum(len(group.slot_pages[s]) for s in (a, b, c))]
        assert ids.tolist() == group.slot_pages[a] + group.slot_pages[b] + group.slot_pages[c]
    assert all(t.dtype == torch.int32 for t in (ctx.token_ids, ctx.tok_pos, ctx.cu_q, ctx.want_rows))
    calls = []
    assert ctx.memo("k", lambda: calls.append(1) or 7) == 7 and ctx.memo("k", lambda: calls.append(1) or 8) == 7
    assert len(calls) == 1


def test_key_split_plan_covers_every_sequence_and_fills_the_gpu_once():
    """Blocks of equal size for unequal sequences: the longest sequence is covered by the splits, no block
    is smaller than asked, and all blocks are on the GPU at once when that can be had."""
    import random

    from ondeviceinfer_b200.kernels.ops import plan_key_splits

    rng = random.Random(5)
    for trial in range(200):
        n = rng.choice([1, 2, 8, 16, 64, 200])
        kv_lens = [rng.randint(1, rng.choice([64, 3000, 140000])) for _ in range(n)]
        rows = rng.choice([1, 2, 8, 16])
        per, splits = plan_key_splits(kv_lens, rows)
        tiles = [-(-k // 64) for k in kv_lens]
        assert per >= 1 and 1 <= splits <= 32
        assert per * splits >= max(tiles)
        assert per >= min(2, max(tiles))
        blocks = sum(-(-t // per) for t in tiles) * rows
        # all blocks on the GPU at once when that can be had; when even whole sequences are too many for that,
        # whole sequences or a few cuts each (which fill the rounds better)
        assert blocks <= 296 or len(tiles) * rows > 296
        if blocks > 296:
            assert per == max(tiles) or splits <= 6
    assert plan_key_splits([2049] * 8, 8) == (9, 4)          # 8 sequences of 33 tiles: four blocks each, 256 in all
    assert plan_key_splits([2049] * 64, 8) == (33, 1)        # more sequences than the GPU holds blocks: each whole
    assert plan_key_splits([2049] * 40, 8) == (11, 3)        # 320 whole sequences would run two rounds for 1.08: three cuts each
    assert plan_key_splits([131001], 8) == (64, 32)          # one long sequence: the most splits there are


def test_the_list_of_key_blocks_covers_every_sequence_within_the_room_fixed_per_width():
    """The decode kernel's grid is as long as the list's room, which depends on the number of sequences alone
    (a graph fixes it): whatever the lengths, the planned blocks fit, every sequence has its blocks 0 .. n-1 with
    the last one marked, and the blocks with the most tiles come first."""
    import random

    import pytest

    from ondeviceinfer_b200.kernels.ops import KernelError, key_split_capacity, key_split_list, plan_key_splits

    rng = random.Random(9)
    for trial in range(300):
        n = rng.choice([1, 2, 5, 8, 16, 37, 38, 40, 64, 200])
        rows = rng.choice([1, 2, 4, 8, 16, 32])
        top = rng.choice([64, 300, 5000, 200000])
        kv_lens = [rng.randint(1, top) for _ in range(n)] if trial % 3 else [rng.randint(1, top)] * n
        per, splits = plan_key_splits(kv_lens, rows)
        room = key_split_capacity(n, rows)
        blocks = key_split_list(kv_lens, per, room)
        assert len(blocks) == 2 + room and blocks[0] == per and blocks[1] <= room
        entries = blocks[2:2 + blocks[1]]
        assert blocks[2 + blocks[1]:] == [0] * (room - blocks[1])
        sizes = []
        for seq, keys in enumerate(kv_lens):
            tiles = -(-keys // 64)
            count = -(-tiles // per)
            assert sorted(e & 255 for e in entries if e >> 8 == seq) == list(range(count - 1)) + [128 | (count - 1)]
            assert count <= splits
        for e in entries:
            tiles = -(-kv_lens[e >> 8] // 64)
            sizes.append(min(per, tiles - (e & 127) * per))
        assert sizes == sorted(sizes, reverse=True) and min(sizes) >= 1
    assert key_split_capacity(8, 8) == 37 and key_split_capacity(64, 8) == 64 * 6 and key_split_capacity(1, 8) == 32
    assert key_split_list([130, 64], 2, 4) == [2, 3, 0 << 8 | 0, 0 << 8 | 128 | 1, 1 << 8 | 128 | 0, 0]
    with pytest.raises(KernelError):
        key_split_list([130, 64], 2, 2)


def test_a_long_step_is_cut_into_passes_of_about_the_token_limit(monkeypatch):
    import importlib
    step = importlib.import_module("ondeviceinfer_b200.engine.step")
    cut = step.tokens_per_sequence_at_a_time
    assert step.STEP_TOKEN_LIMIT == 32768
    assert cut(None, [2048] * 8) is None                       # 16,384 tokens: one pass
    assert cut(None, [8192] * 8) == 4096                       # 65,536 tokens: two passes of 32,768
    assert cut(None, [100000]) == 32768
    assert cut(None, [5000, 40000, 64]) == 10880               # 32,768 // 3 in whole pages
    assert cut(256, [2048] * 8) == 256 and cut(256, [8192] * 8) == 256 and cut(256, [200]) is None
    assert cut(None, [1] * 40000) is None                      # one token each: nothing to cut
    monkeypatch.setattr(step, "STEP_TOKEN_LIMIT", 128)
    assert cut(None, [300, 70, 129]) == 64 and cut(None, [100, 28]) is None and cut(None, [129]) == 128


def test_a_kernel_that_gave_up_waiting_is_reported_once_by_name():
    """Every wait inside the tensor-core kernels is bounded; a kernel whose wait ran out writes a code into
    an error word and returns.  Here the word is set by hand (no GPU is made to wait): the host check names
    the kernel and the role that gave up, clears the word, and is silent afterwards."""
    import pytest
    import torch

    from ondeviceinfer_b200.kernels import ops

    saved = dict(ops._gemm_state)
    try:
        ops._gemm_state.clear()
        ops._gemm_state["test-device"] = {"status": torch.zeros(4, dtype=torch.int32)}
        ops.raise_on_kernel_fault()                                  # nothing happened: no error
        for code, words in ((2, "gemm_tcgen05: the MMA issuer"), (21, "gemm_prefill_tcgen05: the TMA producer"),
                            (13, "attention_tcgen05: the softmax warps")):
            ops._gemm_state["test-device"]["status"][0] = code
            assert ops.gemm_status() == code
            with pytest.raises(ops.KernelError, match=words):
                ops.raise_on_kernel_fault()
            assert ops.gemm_status() == 0
            ops.raise_on_kernel_fault()
    finally:
        ops._gemm_state.clear()
        ops._gemm_state.update(saved)


def test_the_two_step_contexts_give_a_part_the_same_names():
    """A part reads a step through StepDescription.INTERFACE.  The context of the generic step and the
    fixed-buffer context of graph replay both give every one of those names, the generic one gives a part
    nothing else, and what the replay context has beyond them is the runner's own (REPLAY_ONLY): so a part
    written and tested under one cannot break only under the other."""
    from ondeviceinfer_b200.engine.decode import _DecodeContext
    from ondeviceinfer_b200.engine.step import StepDescription

    cache = make_cache()
    a, b = cache.alloc(), cache.alloc()
    cache.reserve([a, b], [3, 1])
    generic = StepContext(cache, [a, b], [[1, 2, 3], [4]], [2, 3], "cpu")
    replay = _DecodeContext(cache, 2, cache.n_pages, "cpu", 256)
    public = lambda obj: {name for name in dir(obj) if not name.startswith("_") and name != "INTERFACE"}
    interface = set(StepDescription.INTERFACE)
    assert interface <= public(generic) and interface <= public(replay) | {"slot_list"}
    assert public(generic) == interface
    assert public(replay) - interface == set(_DecodeContext.REPLAY_ONLY) | {"REPLAY_ONLY"}
    # the mirrors agree in kind: lists of ints per sequence, counts as ints
    for ctx in (generic, replay):
        assert len(ctx.q_lens) == len(ctx.past_lens) == len(ctx.kv_lens) == ctx.n_seqs
        assert [p + q for p, q in zip(ctx.past_lens, ctx.q_lens)] == list(ctx.kv_lens)
        start, ids = ctx.page_table(1)
        assert start.dtype == ids.dtype == torch.int32 and start.numel() == ctx.n_seqs + 1
        assert ctx.memo("k", lambda: 7) == 7 and ctx.memo("k", lambda: 8) == 7
        assert ctx.residual_sumsq is None


def test_generation_stops_with_an_error_when_a_kernel_gave_up_waiting():
    """The generation loop synchronises around the prompts' step and at a batch's end; the entry point's
    synchronise also reads the kernels' error word there.  With the word set by hand during a step the loop
    raises (and gives its slots back) instead of returning tokens computed from an invalid result."""
    from ondeviceinfer_b200.engine.generate import generate_requests
    from ondeviceinfer_b200.kernels import ops

    saved = dict(ops._gemm_state)
    held, steps = set(), []

    def alloc():
        slot = len(held)
        held.add(slot)
        return slot

    def step(slots, runs):
        steps.append(len(steps))
        if len(steps) == 3:                              # a kernel of the third step gives up on a barrier
            ops._gemm_state["test-device"]["status"][0] = 2
        return None

    try:
        ops._gemm_state.clear()
        ops._gemm_state["test-device"] = {"status": torch.zeros(4, dtype=torch.int32)}
        with pytest.raises(ops.KernelError, match="gave up waiting"):
            generate_requests([[1, 2], [3]], max_new_tokens=6, alloc=alloc, free=held.remove, step=step,
                              sample=lambda logits, requests, numbers: [5] * len(requests), batches=[[0, 1]],
                              synchronize=ops.raise_on_kernel_fault)
        assert not held and len(steps) == 6              # the batch ran to its end, then the check refused it
        assert ops.gemm_status() == 0                    # reported once
    finally:
        ops._gemm_state.clear()
        ops._gemm_state.update(saved)


def test_nvtx_ranges_are_off_unless_the_environment_switches_them_on():
    """ONDEVICEINFER_NVTX, read once at import (ondeviceinfer/profiling.py:17-49 of the reference): off, a range
    is the shared do-nothing context; on, it pushes and pops a named range."""
    import subprocess
    import sys

    from ondeviceinfer_b200 import profiling

    assert not profiling.nvtx_enabled()
    assert profiling.nvtx_range("a") is profiling.nvtx_range("b")
    with profiling.nvtx_range("nothing happens"):
        pass
    script = (
        "import torch\n"
        "seen = []\n"
        "torch.cuda.nvtx.range_push = lambda name: seen.append(('push', name))\n"
        "torch.cuda.nvtx.range_pop = lambda: seen.append(('pop',))\n"
        "from ondeviceinfer_b200 import profiling\n"
        "assert profiling.nvtx_enabled()\n"
        "with profiling.nvtx_range('layer_3'):\n"
        "    seen.append(('inside',))\n"
        "assert seen == [('push', 'layer_3'), ('inside',), ('pop',)], seen\n"
        "print('ok')\n")
    import os
    from pathlib import Path
    root = str(Path(__file__).resolve().parent.parent)
    done = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, cwd=root,
                          env=dict(os.environ, ONDEVICEINFER_NVTX="yes", PYTHONPATH=root))
    assert done.returncode == 0 and done.stdout.strip() == "ok", done.stderr
