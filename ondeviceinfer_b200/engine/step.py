"""The step function: run a batch of token runs, one per sequence, from the cache.

A step takes sequences that either all start (their prompts, of unequal lengths) or all
continue (one token each, or a few).  Tokens are packed without padding: sequence ``i``
with ``P_i`` cached positions brings ``T_i`` tokens that sit at positions
``P_i .. P_i + T_i - 1``; their keys and values are appended to the sequence's slot; the
query at position ``p`` sees keys ``0 .. p`` of its own slot only; afterwards the slot's
length is ``P_i + T_i``.  Logits are returned for the wanted places only.

The reference's forward takes a rectangular ``[batch, T]`` block with one past length
shared by the batch (ondeviceinfer/model.py:92-118, ondeviceinfer/cache.py:54); here
every sequence has its own length and its own place in the packed token list.

Everything a kernel needs to know about the step is in :class:`StepContext`, built on the
host and uploaded in one copy.
"""

from __future__ import annotations

import os

from typing import Callable, Dict, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from ..kernels import ops
from ..profiling import nvtx_range

Want = Union[str, Sequence[Sequence[int]]]


class StepDescription:
    """What a part may read from the context of a step, whoever built it.

    Two classes build it: :class:`StepContext` (the host describes a step of any shape and uploads
    it once) and the fixed-buffer context of :mod:`ondeviceinfer_b200.engine.decode` (one token per
    sequence, replayed as a CUDA graph).  ``INTERFACE`` names everything both give; a part written
    against these names runs under either (a test holds the two to it).  All index tensors are int32.

    ``token_ids [n_tokens]``  the packed tokens;
    ``tok_seq [n_tokens]``    index (within the batch) of each token's sequence;
    ``tok_pos [n_tokens]``    absolute position of each token in its sequence;
    ``cu_q [n_seqs + 1]``     first packed token of each sequence;
    ``past [n_seqs]``         cached length of each sequence before the step;
    ``slots [n_seqs]``        cache slot of each sequence (row of the state tensors);
    ``want_rows [n_want]``    packed token indices whose logits are returned;
    ``page_table(g)``         ``(page_start [n_seqs + 1], page_ids)`` of key/value group g;
    ``key_splits(rows)``      how a split-key decode kernel may cut the sequences' keys;
    ``memo(key, make)``       a value shared by all layers of the step (rotary tables and the like);
    ``residual_sumsq``        the note a residual product leaves for the norm that follows it;
    ``pending_residual_add``, ``defers_residual_add``  a residual add left to the next norm, and the flag of a block
                              that finishes such adds (``parts/linear.py``, ``parts/block.py``).

    Host mirrors: ``n_seqs``, ``n_tokens``, ``n_want``, ``q_lens``, ``past_lens``, ``kv_lens`` (keys each
    sequence sees after the step), ``max_q_len``, ``max_kv_len``, ``slot_list``.  Under graph replay the host
    code of a part runs at capture only: a part that is marked ``graph_safe`` lets the mirrors decide sizes
    and kernel forms (which a graph fixes, and for which the runner keeps one graph per width and length
    bucket), never values.
    """

    INTERFACE = ("token_ids", "tok_seq", "tok_pos", "cu_q", "past", "slots", "want_rows",
                 "n_seqs", "n_tokens", "n_want", "q_lens", "past_lens", "kv_lens", "max_q_len", "max_kv_len",
                 "slot_list", "residual_sumsq", "pending_residual_add", "defers_residual_add",
                 "page_table", "key_splits", "memo")

    def __init__(self) -> None:
        self._memo: Dict[object, object] = {}
        self._page_tables: List[Tuple[torch.Tensor, torch.Tensor]] = []
        self.residual_sumsq = None
        self.pending_residual_add = None       # (residual, product) that a block left to the next norm
        self.defers_residual_add = False       # set by a block that finishes such adds

    def page_table(self, group_index: int) -> Tuple[torch.Tensor, torch.Tensor]:
        return self._page_tables[group_index]

    def memo(self, key, make: Callable[[], object]):
        """A value shared by all layers of the step (rotary tables and the like)."""
        if key not in self._memo:
            self._memo[key] = make()
        return self._memo[key]

    @property
    def kv_lens(self) -> List[int]:
        return [p + t for p, t in zip(self.past_lens, self.q_lens)]

    def key_splits(self, block_rows: int) -> Tuple[Optional[torch.Tensor], int]:
        raise NotImplementedError


class StepContext(StepDescription):
    """Device-side description of a step, built on the host and uploaded in one copy
    (fields: see :class:`StepDescription`)."""

    def __init__(self, cache, slots: Sequence[int], tokens: Sequence[Sequence[int]],
                 want_rows: Sequence[int], device) -> None:
        super().__init__()
        self.n_seqs = len(slots)
        self.slot_list = list(slots)
        self.q_lens = [len(t) for t in tokens]
        self.past_lens = [cache.lengths[s] for s in slots]
        self.n_tokens = sum(self.q_lens)
        self.max_q_len = max(self.q_lens)
        self.max_kv_len = max(p + t for p, t in zip(self.past_lens, self.q_lens))
        self.n_want = len(want_rows)

        q = np.asarray(self.q_lens, dtype=np.int64)
        cu = np.zeros(self.n_seqs + 1, dtype=np.int64)
        np.cumsum(q, out=cu[1:])
        past = np.asarray(self.past_lens, dtype=np.int64)
        tok_seq = np.repeat(np.arange(self.n_seqs), q)
        tok_pos = np.arange(self.n_tokens) - np.repeat(cu[:-1], q) + np.repeat(past, q)
        ids = np.fromiter((t for run in tokens for t in run), dtype=np.int64, count=self.n_tokens)
        pieces = [ids, tok_seq, tok_pos, cu, past, np.asarray(slots, dtype=np.int64),
                  np.asarray(want_rows, dtype=np.int64)]
        for group in cache.kv_groups:
            lists = [group.slot_pages[s] for s in slots]
            start = np.zeros(self.n_seqs + 1, dtype=np.int64)
            np.cumsum([len(l) for l in lists], out=start[1:])
            pieces += [start, np.fromiter((p for l in lists for p in l), dtype=np.int64, count=int(start[-1]))]
        sizes = [len(p) for p in pieces]
        packed = np.concatenate(pieces).astype(np.int32)
        self._meta = torch.from_numpy(packed).to(device)
        views, offset = [], 0
        for size in sizes:
            views.append(self._meta[offset:offset + size])
            offset += size
        (self.token_ids, self.tok_seq, self.tok_pos, self.cu_q, self.past, self.slots, self.want_rows) = views[:7]
        self._page_tables = [(views[7 + 2 * g], views[8 + 2 * g]) for g in range(len(cache.kv_groups))]

    def key_splits(self, block_rows: int) -> Tuple[Optional[torch.Tensor], int]:
        """For a mixer whose decode kernel cuts each sequence's keys among blocks (``block_rows`` blocks per
        cut): ``(tiles_per_split, splits)`` as :func:`ondeviceinfer_b200.kernels.ops.plan_key_splits` gives
        them for this step's sequences, the first on the device as the kernel's list of blocks
        (:func:`ondeviceinfer_b200.kernels.ops.key_split_list`)."""
        def make():
            per, splits = ops.plan_key_splits(self.kv_lens, block_rows)
            blocks = ops.key_split_list(self.kv_lens, per, ops.key_split_capacity(len(self.kv_lens), block_rows))
            return torch.tensor(blocks, dtype=torch.int32).to(self.past.device, non_blocking=True), splits
        return self.memo(("key_splits", block_rows), make)


def resolve_want(want: Want, q_lens: Sequence[int]) -> List[List[int]]:
    """Per sequence, the places (indices into this step's tokens) whose logits are wanted."""
    if isinstance(want, str):
        if want == "last":
            return [[t - 1] for t in q_lens]
        if want == "all":
            return [list(range(t)) for t in q_lens]
        if want == "none":
            return [[] for _ in q_lens]
        raise ValueError(f"want must be 'last', 'all', 'none' or a list of places per sequence, not {want!r}")
    places = [list(w) for w in want]
    if len(places) != len(q_lens):
        raise ValueError(f"want names {len(places)} sequences, the step has {len(q_lens)}")
    for i, (w, t) in enumerate(zip(places, q_lens)):
        for place in w:
            if not 0 <= place < t:
                raise ValueError(f"sequence {i} brings {t} tokens, place {place} is outside them")
    return places


def validate_step(cache, slots: Sequence[int], tokens: Sequence[Sequence[int]], vocab_size: int) -> None:
    if len(slots) != len(tokens):
        raise ValueError(f"{len(slots)} slots but {len(tokens)} token runs")
    if not slots:
        raise ValueError("a step needs at least one sequence")
    if len(set(slots)) != len(slots):
        raise ValueError(f"a slot appears twice in the batch: {list(slots)}")
    for i, (slot, run) in enumerate(zip(slots, tokens)):
        if not cache.slots.is_held(slot):
            raise ValueError(f"sequence {i}: slot {slot} is not held")
        if len(run) == 0:
            raise ValueError(f"sequence {i} brings no tokens")
        lo, hi = min(run), max(run)
        if lo < 0 or hi >= vocab_size:
            raise ValueError(f"sequence {i}: token id {lo if lo < 0 else hi} is outside the vocabulary of {vocab_size}")


# The most tokens that one pass over the layers takes (ODI_STEP_TOKENS).  Longer steps run as several passes
# over the same cache, which bounds the activations (a pass of 32,768 tokens of Qwen3-8B's width holds under
# 2 GB of them) and keeps every index inside a kernel well below 2^31, and costs nothing: the many-token
# kernels are at their full rate from a few thousand tokens on.
STEP_TOKEN_LIMIT = int(os.environ.get("ODI_STEP_TOKENS", "32768"))


def tokens_per_sequence_at_a_time(cache_limit: Optional[int], q_lens: Sequence[int]) -> Optional[int]:
    """How many tokens of each sequence one pass takes, or None if the whole step is one pass.  A cache with
    windowed groups takes at most ``cache_limit`` per sequence at a time (its rings are sized for that); a step of
    more than ``STEP_TOKEN_LIMIT`` tokens is cut so that a pass holds about that many, in whole pages of 64."""
    limit = cache_limit
    if sum(q_lens) > STEP_TOKEN_LIMIT:
        share = max(64, STEP_TOKEN_LIMIT // len(q_lens) // 64 * 64)
        limit = share if limit is None else min(limit, share)
    return None if limit is None or max(q_lens) <= limit else limit


def run_step(model, cache, slots: Sequence[int], tokens: Sequence[Sequence[int]], want: Want = "last") -> torch.Tensor:
    """Run one step and return fp32 logits ``[n_wanted, vocab]`` on the device, ordered by
    sequence and then by place.  See the module text for the contract."""
    tokens = [list(run) for run in tokens]
    validate_step(cache, slots, tokens, model.vocab_size)
    places = resolve_want(want, [len(t) for t in tokens])
    limit = tokens_per_sequence_at_a_time(cache.max_step_tokens, [len(t) for t in tokens])
    if limit is None:
        return _run_chunk(model, cache, slots, tokens, places)
    # Cut the step into sub-steps of at most `limit` tokens per sequence and put the wanted rows back in order.
    outputs: List[List[Optional[torch.Tensor]]] = [[None] * len(p) for p in places]
    offset = 0
    while True:
        part_slots, part_tokens, part_places, origin = [], [], [], []
        for i, run in enumerate(tokens):
            piece = run[offset:offset + limit]
            if not piece:
                continue
            part_slots.append(slots[i])
            part_tokens.append(piece)
            here = [(j, p - offset) for j, p in enumerate(places[i]) if offset <= p < offset + limit]
            part_places.append([p for _, p in here])
            origin.append([(i, j) for j, _ in here])
        if not part_slots:
            break
        logits = _run_chunk(model, cache, part_slots, part_tokens, part_places)
        row = 0
        for seq in origin:
            for (i, j) in seq:
                outputs[i][j] = logits[row]
                row += 1
        offset += limit
    rows = [r for seq in outputs for r in seq]
    if not rows:
        return torch.empty((0, getattr(model, "logits_size", model.vocab_size)), dtype=torch.float32, device=model.device)
    return torch.stack(rows)


def _run_chunk(model, cache, slots, tokens, places) -> torch.Tensor:
    q_lens = [len(t) for t in tokens]
    cache.reserve(slots, q_lens)
    starts = np.concatenate(([0], np.cumsum(q_lens)[:-1])) if q_lens else []
    want_rows = [int(starts[i]) + p for i, seq in enumerate(places) for p in seq]
    with nvtx_range(f"step[{len(slots)} seqs, {sum(q_lens)} tokens]"):
        ctx = StepContext(cache, slots, tokens, want_rows, model.device)
        logits = model.forward(ctx, cache)
    cache.advance(slots, q_lens)
    return logits
