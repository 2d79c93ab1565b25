"""Decode steps as CUDA graphs: one token per live sequence per replay, nothing rebuilt on the host.

The generic step function builds its index tensors on the host and launches some three
hundred kernels from Python; for single-token steps that costs several times what the
GPU needs.  A :class:`DecodeRunner` keeps the step's index tensors in fixed device
buffers, captures embedding -> layers -> head -> sampling once per batch width as a CUDA
graph, and replays it: the sampled token is written where the next step reads its
input, and the sampling kernel advances positions, lengths and step numbers in place.
Per step the host only makes sure every sequence has a page for its next position and
chooses the graph.

What a graph fixes besides the width: how a mixer's decode kernel may cut a sequence's keys
among blocks.  That follows the sequences' lengths, so there is one graph per power of two of
the longest sequence and per bound on the number of cuts (a power of two as well); all graphs of
a width share its buffers, and a batch that outgrows its graph in the middle goes on with
another.  The size of the cuts and the list of (sequence, cut) blocks that follow from it live on
the device in a buffer of the width; the host refreshes them when a sequence enters another tile of
64 keys (:meth:`_DecodeContext.plan_key_splits`).

Widths are powers of two up to 32, then multiples of 16; rows beyond the live sequences are padding: they run on a
slot outside the cache's capacity with a constant length of zero and their results are dropped, so
padding changes no result.  The same kernels run as in the generic step; only the way
they are launched differs.  Models with parts that do host work per step (anything that
is not marked ``graph_safe``) do not use this path.
"""

from __future__ import annotations

import gc
import time
import weakref
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..kernels import ops
from ..profiling import nvtx_range
from .step import StepDescription


def _power_of_two(n: int) -> int:
    p = 1
    while p < n:
        p *= 2
    return p


def serving_graph_key(keys, width: int, bucket: int, bounds: tuple):
    """Which of the captured graphs ``keys`` (each ``(width, longest-sequence bucket, bounds on the key splits)``)
    serves a step that needs ``(width, bucket, bounds)``: the very one, else the smallest made for sequences up to
    twice as long and for up to twice the splits (its surplus blocks leave at once, and a capture costs what
    hundreds of steps take), else None."""
    if (width, bucket, bounds) in keys:
        return (width, bucket, bounds)
    near = [k for k in keys
            if k[0] == width and bucket <= k[1] <= 2 * bucket and len(k[2]) == len(bounds)
            and all(need <= have <= 2 * need for need, have in zip(bounds, k[2]))]
    return min(near, key=lambda k: (k[1], k[2])) if near else None


class _DecodeContext(StepDescription):
    """The fixed-buffer counterpart of :class:`~ondeviceinfer_b200.engine.step.StepContext`
    for ``width`` sequences that bring one token each: the same names for a part
    (:class:`~ondeviceinfer_b200.engine.step.StepDescription`), plus what only the runner uses
    (``REPLAY_ONLY``)."""

    REPLAY_ONLY = ("width", "max_pages", "streams", "steps", "active", "plan_key_splits")

    def __init__(self, cache, width: int, max_pages: int, device, longest: int) -> None:
        super().__init__()
        self.width = width
        self.n_seqs = self.n_tokens = self.n_want = width
        self.max_q_len = 1
        self.q_lens = [1] * width
        self.max_kv_len = longest
        self.max_pages = max_pages
        arange = torch.arange(width + 1, dtype=torch.int32, device=device)
        zeros = lambda n: torch.zeros(n, dtype=torch.int32, device=device)
        self.token_ids, self.tok_pos, self.past, self.slots = zeros(width), zeros(width), zeros(width), zeros(width)
        self.streams, self.steps, self.active = zeros(width), zeros(width), zeros(width)
        self.tok_seq = arange[:width].clone()
        self.want_rows = arange[:width].clone()
        self.cu_q = arange.clone()
        page_start = (arange * max_pages).contiguous()
        self._page_ids = [zeros(width * max_pages) for _ in cache.kv_groups]
        self._page_tables = [(page_start, ids) for ids in self._page_ids]
        self.slot_list: List[int] = []
        self._kv_lens: List[int] = [longest] * width         # host: the keys each row sees in the coming step
        self._key_splits: Dict[int, list] = {}               # block rows -> [the list on the device, on the host, bound on the splits]
        self._planned_tiles: tuple = ()
        self._planned_bounds: tuple = ()

    @property
    def kv_lens(self) -> List[int]:
        return self._kv_lens

    @kv_lens.setter
    def kv_lens(self, values: Sequence[int]) -> None:
        self._kv_lens = list(values)

    @property
    def past_lens(self) -> List[int]:
        return [n - 1 for n in self._kv_lens]

    def key_splits(self, block_rows: int):
        """``(tiles_per_split, splits)`` for a mixer whose decode kernel cuts each sequence's keys among
        blocks.  The first is the kernel's list of blocks on the device
        (:func:`~ondeviceinfer_b200.kernels.ops.key_split_list`, as long as any plan for this width can make it),
        which :meth:`plan_key_splits` refreshes before a replay; the second, a power of two, is fixed in the
        graph being captured."""
        if block_rows not in self._key_splits:
            per, splits = ops.plan_key_splits(self.kv_lens, block_rows)
            blocks = ops.key_split_list(self.kv_lens, per, ops.key_split_capacity(self.width, block_rows))
            self._key_splits[block_rows] = [torch.tensor(blocks, dtype=torch.int32, device=self.token_ids.device), blocks,
                                            _power_of_two(splits)]
        entry = self._key_splits[block_rows]
        return entry[0], entry[2]

    def plan_key_splits(self, kv_lens: Sequence[int], fix_bounds: bool = False) -> tuple:
        """Refresh the lists of blocks for the coming step and return the bounds on the splits that it needs,
        as a key for the graph to replay; ``fix_bounds`` makes them the bounds of the next capture."""
        tiles = tuple(-(-n // 64) for n in kv_lens)
        if tiles == self._planned_tiles and not fix_bounds and len(self._planned_bounds) == len(self._key_splits):
            return self._planned_bounds           # the plan only changes when a sequence enters another tile
        self.kv_lens = list(kv_lens)
        needed = []
        for block_rows in sorted(self._key_splits):
            entry = self._key_splits[block_rows]
            per, splits = ops.plan_key_splits(self.kv_lens, block_rows)
            blocks = ops.key_split_list(self.kv_lens, per, entry[0].numel() - 2)
            if blocks != entry[1]:
                # from pageable memory: the copy has left the host's list when the call returns, and is
                # ordered on the stream before the replay that reads it
                entry[0].copy_(torch.tensor(blocks, dtype=torch.int32))
                entry[1] = blocks
            needed.append(_power_of_two(splits))
            if fix_bounds:
                entry[2] = needed[-1]
        self._planned_tiles, self._planned_bounds = tiles, tuple(needed)
        return self._planned_bounds


class DecodeRunner:
    def __init__(self, model, cache, *, temperature: float = 0.0, seed: int = 0) -> None:
        # The cache keeps its runners (ondeviceinfer_b200.api.decode_runner); the runner must not keep the cache
        # alive in turn, or the two, and the runner's graphs, would only go when the cycle collector runs:
        # possibly in the middle of another capture, which a graph's destruction invalidates.
        self.model, self._cache = model, weakref.ref(cache)
        self.temperature, self.seed = float(temperature), int(seed)
        self.max_pages = cache.n_pages
        self._contexts: Dict[int, _DecodeContext] = {}     # by width: the buffers that every graph of the width uses
        self._graphs: Dict[tuple, tuple] = {}               # by (width, longest-sequence bucket, split bounds)
        self._last_key: Optional[tuple] = None              # the graph that the last step replayed
        self.capture_seconds = 0.0                          # wall time spent capturing graphs so far
        self.live_slots: List[int] = []
        self.ctx: Optional[_DecodeContext] = None
        self._host_pages: List[np.ndarray] = []
        self._pinned_tokens: Optional[torch.Tensor] = None
        self._pinned_out: Optional[torch.Tensor] = None

    @property
    def cache(self):
        cache = self._cache()
        if cache is None:
            raise RuntimeError("the cache of this decode runner is gone")
        return cache

    # ------------------------------------------------------------------ set-up

    def close(self) -> None:
        self._graphs.clear()
        self._contexts.clear()

    @staticmethod
    def _bucket_for(kv_len: int) -> int:
        """A captured graph fixes how the keys of a sequence are cut among blocks, which is chosen from
        the longest sequence: one graph per power of two of that length, from 256 on."""
        bucket = 256
        while bucket < kv_len:
            bucket *= 2
        return bucket

    @staticmethod
    def _width_for(n: int) -> int:
        """Captured widths: powers of two up to 32, then multiples of 16 (the padding rows cost a full
        row of every kernel, so a batch of 33 should not run as 64)."""
        if n > 32:
            return -(-n // 16) * 16
        width = 1
        while width < n:
            width *= 2
        return width

    def begin(self, slots: Sequence[int], tokens: Sequence[int], streams: Sequence[int], steps: Sequence[int]) -> None:
        """Make ``slots`` the live set: sequence i will be fed ``tokens[i]`` next; ``streams``
        and ``steps`` are its request index and the number of tokens it has produced so far."""
        n = len(slots)
        if n == 0:
            raise ValueError("a decode batch needs at least one sequence")
        width = self._width_for(n)
        self._graph_for(width, [self.cache.lengths[s] + 1 for s in slots])
        ctx = self._contexts[width]
        self.ctx, self.live_slots = ctx, list(slots)
        pad = self.cache.pad_slot
        row_slots = list(slots) + [pad] * (width - n)
        lengths = [self.cache.lengths[s] for s in slots] + [0] * (width - n)
        fill = lambda values: torch.tensor(list(values) + [0] * (width - len(values)), dtype=torch.int32)
        host = torch.stack([fill(tokens), torch.tensor(lengths, dtype=torch.int32), torch.tensor(row_slots, dtype=torch.int32),
                            fill(streams), fill(steps), fill([1] * n)]).to(self.model.device)
        ctx.token_ids.copy_(host[0]); ctx.tok_pos.copy_(host[1]); ctx.past.copy_(host[1]); ctx.slots.copy_(host[2])
        ctx.streams.copy_(host[3]); ctx.steps.copy_(host[4]); ctx.active.copy_(host[5])
        ctx.slot_list = row_slots
        self._host_pages = []
        for g, group in enumerate(self.cache.kv_groups):
            table = np.zeros((width, self.max_pages), dtype=np.int32)
            for i, slot in enumerate(row_slots):
                pages = group.slot_pages[slot]
                table[i, :len(pages)] = pages
            self._host_pages.append(table)
            ctx._page_ids[g].copy_(torch.from_numpy(table.reshape(-1)))

    def _reserve_next(self, ahead: int = 1) -> None:
        """Pages for the next ``ahead`` positions of every live sequence; upload what changed."""
        n = len(self.live_slots)
        before = [[len(g.slot_pages[s]) for s in self.live_slots] for g in self.cache.kv_groups]
        self.cache.reserve(self.live_slots, [ahead] * n)
        for g, group in enumerate(self.cache.kv_groups):
            for i, slot in enumerate(self.live_slots):
                pages = group.slot_pages[slot]
                if len(pages) != before[g][i]:
                    self._host_pages[g][i, :len(pages)] = pages
                    lo = i * self.max_pages + before[g][i]
                    self.ctx._page_ids[g][lo:lo + len(pages) - before[g][i]].copy_(
                        torch.tensor(pages[before[g][i]:], dtype=torch.int32))

    # ------------------------------------------------------------------ capture

    def _run_once(self, ctx: _DecodeContext) -> torch.Tensor:
        ctx._memo.clear()
        ctx.residual_sumsq = None
        logits = self.model.forward(ctx, self.cache)
        ops.sample(logits, ctx.token_ids, self.temperature, self.seed, ctx.streams, ctx.steps,
                   advance_pos=ctx.tok_pos, advance_past=ctx.past, active=ctx.active)
        return logits

    def _graph_for(self, width: int, kv_lens: Sequence[int]):
        """The graph for ``width`` rows whose live sequences see ``kv_lens`` keys in the coming step: one per
        power of two of the longest sequence and per bound on the key splits; padding rows see one key."""
        kv_lens = list(kv_lens) + [1] * (width - len(kv_lens))
        bucket = self._bucket_for(max(kv_lens))
        ctx = self._contexts.get(width)
        if ctx is None:
            ctx = self._contexts[width] = _DecodeContext(self.cache, width, self.max_pages, self.model.device, bucket)
            ctx.kv_lens = kv_lens
            graph = self._capture(ctx, bucket)          # its warm-up run tells which parts cut keys
            self._last_key = (width, bucket, ctx.plan_key_splits(kv_lens))
            self._graphs[self._last_key] = graph
            return graph
        key = (width, bucket, ctx.plan_key_splits(kv_lens))
        have = serving_graph_key(self._graphs, *key)
        if have is not None:
            self._last_key = have
            return self._graphs[have]
        # in the middle of a batch: the capture runs on the pad slot and overwrites the buffers
        names = ("token_ids", "tok_pos", "past", "slots", "streams", "steps", "active")
        saved = [getattr(ctx, name).clone() for name in names]
        pages = [ids.clone() for ids in ctx._page_ids]
        slot_list = ctx.slot_list
        ctx.plan_key_splits(kv_lens, fix_bounds=True)
        self._graphs[key] = self._capture(ctx, bucket)
        for name, value in zip(names, saved):
            getattr(ctx, name).copy_(value)
        for ids, value in zip(ctx._page_ids, pages):
            ids.copy_(value)
        ctx.slot_list = slot_list
        self._last_key = key
        return self._graphs[key]

    def _capture(self, ctx: _DecodeContext, bucket: int):
        device, width = self.model.device, ctx.width
        torch.cuda.synchronize(device)
        began = time.perf_counter()
        with nvtx_range(f"capture[{width} rows, up to {bucket} keys]"):
            return self._capture_now(ctx, bucket, device, width, began)

    def _capture_now(self, ctx: _DecodeContext, bucket: int, device, width: int, began: float):
        ctx.max_kv_len = bucket
        pad = self.cache.pad_slot
        ctx.slots.fill_(pad)
        ctx.slot_list = [pad] * width
        for g, group in enumerate(self.cache.kv_groups):
            ctx._page_ids[g].fill_(group.slot_pages[pad][0])
        # The rows' lengths as the plan has them: the list of key blocks on the device was made for these, and a
        # kernel that finds longer sequences than its list covers reports it.  (The buffers may still hold the
        # lengths of an earlier, longer batch.)  Wherever a position points, the run reads and writes the pad
        # slot's one page.
        planned = torch.tensor([max(int(n) - 1, 0) for n in ctx.kv_lens], dtype=torch.int32)
        ctx.past.copy_(planned)
        ctx.tok_pos.copy_(planned)
        # The run before the capture compiles, sizes scratch, sets function attributes and loads every kernel
        # that the graph will hold: a kernel's first launch is not allowed inside a capture, and a graph for
        # more key splits may be the first to use one (the merge of the splits).
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            self._run_once(ctx)
        torch.cuda.current_stream(device).wait_stream(side)
        torch.cuda.synchronize(device)
        ops.raise_on_kernel_fault()          # what this run reports belongs to it, not to the next step
        ctx.tok_pos.zero_(); ctx.past.zero_(); ctx.steps.zero_()
        counted = dict(ops.LAUNCHES)
        graph = torch.cuda.CUDAGraph()
        # No cycle collection while the stream captures: it could destroy a dropped graph of somebody else's,
        # which is not allowed then and invalidates this capture.  What is garbage already goes first.
        gc.collect()
        collecting = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(graph):
                logits = self._run_once(ctx)
        finally:
            if collecting:
                gc.enable()
        launches = {k: ops.LAUNCHES[k] - counted[k] for k in ("own", "library")}
        ctx.tok_pos.zero_(); ctx.past.zero_(); ctx.steps.zero_()
        torch.cuda.synchronize(device)
        self.capture_seconds += time.perf_counter() - began
        # `logits` lives in the graph's own memory: every replay of this graph leaves the step's logits there
        return graph, launches, logits

    # ------------------------------------------------------------------ steps

    def step_device(self, n_steps: int = 1) -> None:
        """Replay ``n_steps`` decode steps back to back; tokens stay on the device."""
        self._reserve_next(n_steps)
        lengths = [self.cache.lengths[s] for s in self.live_slots]
        for i in range(n_steps):
            graph, launches, _ = self._graph_for(self.ctx.width, [n + i + 1 for n in lengths])
            with nvtx_range(f"decode_step[{self.ctx.width} rows]"):
                graph.replay()
            ops.LAUNCHES["own"] += launches["own"]
            ops.LAUNCHES["library"] += launches["library"]
        self.cache.advance(self.live_slots, [n_steps] * len(self.live_slots))

    def step(self, host_tokens: Optional[Sequence[int]] = None) -> List[int]:
        """One decode step; returns the sampled tokens of the live sequences.  With
        ``host_tokens`` the step's inputs are first copied from pinned host memory."""
        n = len(self.live_slots)
        if host_tokens is not None:
            if self._pinned_tokens is None or self._pinned_tokens.numel() < n:
                self._pinned_tokens = torch.empty(max(n, 64), dtype=torch.int32).pin_memory()
            self._pinned_tokens[:n] = torch.as_tensor(host_tokens, dtype=torch.int32)
            self.ctx.token_ids[:n].copy_(self._pinned_tokens[:n], non_blocking=True)
        self.step_device(1)
        # the sampled tokens back through pinned memory, and with them the kernels' error word: two asynchronous
        # copies, one wait on the stream
        if self._pinned_out is None or self._pinned_out.numel() < n + 1:
            self._pinned_out = torch.empty(max(n, 64) + 1, dtype=torch.int32).pin_memory()
        self._pinned_out[:n].copy_(self.ctx.token_ids[:n], non_blocking=True)
        self._pinned_out[n:n + 1].copy_(ops.kernel_status_word(self.model.device), non_blocking=True)
        torch.cuda.current_stream().synchronize()
        if int(self._pinned_out[n]) != 0:
            ops.raise_on_kernel_fault()
        return self._pinned_out[:n].tolist()

    def last_logits(self) -> torch.Tensor:
        """fp32 logits ``[live sequences, vocab]`` of the step replayed last, on the device: a view of the
        memory the replayed graph writes them to, valid until the next step."""
        if self._last_key is None:
            raise RuntimeError("no decode step has run yet")
        return self._graphs[self._last_key][2][:len(self.live_slots)]

    def drop(self, finished_rows: Sequence[int], streams: Sequence[int], steps: Sequence[int]) -> None:
        """Remove rows (indices into the live set) and continue with the others; ``streams``
        and ``steps`` describe the sequences that stay, in order."""
        keep = [i for i in range(len(self.live_slots)) if i not in set(finished_rows)]
        if not keep:
            self.live_slots = []
            return
        tokens = self.ctx.token_ids[:len(self.live_slots)].tolist()
        self.begin([self.live_slots[i] for i in keep], [tokens[i] for i in keep], streams, steps)
