"""The cache of a model: a slot per live sequence, paged keys and values per layer, and
fixed-size per-sequence state.

* A **slot** is what a sequence holds from its first token to its end: its length, its
  pages in every key/value group, and its row in every state tensor.  Slots are taken
  with :meth:`SequenceCache.alloc` and given back with :meth:`SequenceCache.free`;
  a freed slot and its pages are used again by later sequences.
* Keys and values live in **pages** of :data:`PAGE_SIZE` positions.  The capacity of the
  cache is a number of tokens: the sum over live sequences of their lengths, each
  rounded up to a whole page.  (The reference preallocates a rectangle
  ``[batch, kv_heads, max_seq_len, head_dim]`` per layer with one length shared by the
  whole batch, ondeviceinfer/cache.py:51-54; pages let sequences of unequal length share
  one pool, and each sequence has its own length.)
* Layers whose mixers ask for the same thing form a **group** with storage of its own:
  all layers that keep every key (``KVNeed`` without window), all layers that keep a
  window of the same size, all layers with the same ``StateNeed``.  A windowed group
  keeps a ring of pages per sequence instead of all of them.
* The layout of a key/value pool is ``[owner, 2, page, kv_head, row, head_dim]``
  (owner = a layer execution that writes its own cache; 2 = keys, values), so one
  (page, head) tile is a dense ``[PAGE_SIZE, head_dim]`` box.

Errors follow ondeviceinfer/cache.py:65-75 in spirit: capacity exceeded, unknown slot.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .allocators import CacheCapacityError, IndexAllocator
from .needs import KVNeed, StateNeed

PAGE_SIZE = 64


def pages_for(tokens: int) -> int:
    return (tokens + PAGE_SIZE - 1) // PAGE_SIZE


class KVGroup:
    """Storage of the layer executions that share one :class:`KVNeed`."""

    def __init__(self, index: int, need: KVNeed, owners: List[int], n_pages: int, n_slots: int,
                 dtype: torch.dtype, device, max_step_tokens: int) -> None:
        self.index, self.need, self.owners = index, need, owners
        if need.window is None:
            self.ring_pages = 0
        else:
            # positions [p - window + 1, p + step - 1] must map to distinct rows of the ring
            self.ring_pages = pages_for(need.window + max_step_tokens - 1) + 1
        # one page and one slot beyond the capacity belong to padding rows of fixed-width steps
        self.pool = torch.zeros((len(owners), 2, n_pages + 1, need.num_kv_heads, PAGE_SIZE, need.head_dim),
                                dtype=dtype, device=device)
        self.pages = IndexAllocator(n_pages, "page")
        self.pad_page = n_pages
        self.slot_pages: List[List[int]] = [[] for _ in range(n_slots)] + [[self.pad_page]]

    def pages_needed(self, length: int) -> int:
        n = pages_for(length)
        return n if self.ring_pages == 0 else min(n, self.ring_pages)

    def keys(self, owner_pos: int) -> torch.Tensor:
        return self.pool[owner_pos, 0]

    def values(self, owner_pos: int) -> torch.Tensor:
        return self.pool[owner_pos, 1]


class StateGroup:
    def __init__(self, index: int, need: StateNeed, owners: List[int], n_slots: int, device) -> None:
        self.index, self.need, self.owners = index, need, owners
        self.data = torch.zeros((len(owners), n_slots + 1) + tuple(need.shape), dtype=need.dtype, device=device)


@dataclass
class CacheView:
    """What one layer execution sees of the cache."""

    kv_group: Optional[KVGroup] = None
    keys: Optional[torch.Tensor] = None      # [pages, kv_heads, PAGE_SIZE, head_dim]
    values: Optional[torch.Tensor] = None
    writes_kv: bool = True                   # False: reads the cache another execution wrote
    state: Optional[torch.Tensor] = None     # [slots, *shape]


class SequenceCache:
    """``needs[e]`` is the tuple of needs of order entry ``e`` (empty for an entry that
    reads another entry's cache); ``cache_from[e]`` names that other entry or is None."""

    def __init__(self, needs: Sequence[Tuple[object, ...]], cache_from: Sequence[Optional[int]], *,
                 dtype: torch.dtype, device, max_tokens: int, max_seqs: int,
                 max_step_tokens: int = 256) -> None:
        if max_tokens <= 0:
            raise ValueError("max_tokens must be positive")
        if max_seqs <= 0:
            raise ValueError("max_seqs must be positive")
        self.dtype, self.device = dtype, torch.device(device)
        self.max_tokens, self.max_seqs = max_tokens, max_seqs
        self.n_pages = pages_for(max_tokens)
        self.slots = IndexAllocator(max_seqs, "slot")
        self.lengths = [0] * (max_seqs + 1)
        # A slot outside the capacity, of constant length 0, with one page of its own in every
        # group: rows that only pad a fixed-width batch run on it and their results are dropped.
        self.pad_slot = max_seqs
        self.kv_groups: List[KVGroup] = []
        self.state_groups: List[StateGroup] = []
        self._views: List[CacheView] = []

        kv_owners: Dict[KVNeed, List[int]] = {}
        state_owners: Dict[StateNeed, List[int]] = {}
        for entry, entry_needs in enumerate(needs):
            if cache_from[entry] is not None:
                continue
            for need in entry_needs:
                if isinstance(need, KVNeed):
                    kv_owners.setdefault(need, []).append(entry)
                elif isinstance(need, StateNeed):
                    state_owners.setdefault(need, []).append(entry)
                else:
                    raise TypeError(f"order entry {entry}: unknown cache need {need!r}")
        self.has_window = any(n.window is not None for n in kv_owners)
        self.max_step_tokens = max_step_tokens if self.has_window else None
        for need, owners in kv_owners.items():
            self.kv_groups.append(KVGroup(len(self.kv_groups), need, owners, self.n_pages, max_seqs,
                                          dtype, device, max_step_tokens))
        for need, owners in state_owners.items():
            self.state_groups.append(StateGroup(len(self.state_groups), need, owners, max_seqs, device))

        for entry in range(len(needs)):
            source = entry if cache_from[entry] is None else cache_from[entry]
            view = CacheView(writes_kv=cache_from[entry] is None)
            for group in self.kv_groups:
                if source in group.owners:
                    if view.kv_group is not None:
                        raise ValueError(f"order entry {source} asks for two key/value stores")
                    pos = group.owners.index(source)
                    view.kv_group, view.keys, view.values = group, group.keys(pos), group.values(pos)
            for group in self.state_groups:
                if source in group.owners:
                    view.state = group.data[group.owners.index(source)]
            self._views.append(view)

    # ------------------------------------------------------------------ slots

    def alloc(self) -> int:
        """A free slot with length 0 and zeroed state."""
        slot = self.slots.take()
        self.lengths[slot] = 0
        for group in self.state_groups:
            group.data[:, slot].zero_()
        return slot

    def free(self, slot: int) -> None:
        """Give the slot and all its pages back."""
        if not self.slots.is_held(slot):
            raise ValueError(f"slot {slot} is not held (freed twice, or never allocated)")
        for group in self.kv_groups:
            for page in group.slot_pages[slot]:
                group.pages.give_back(page)
            group.slot_pages[slot] = []
        self.lengths[slot] = 0
        self.slots.give_back(slot)

    def reset(self) -> None:
        for slot in range(self.max_seqs):
            if self.slots.is_held(slot):
                self.free(slot)

    def length(self, slot: int) -> int:
        self._require_held(slot)
        return self.lengths[slot]

    def _require_held(self, slot: int) -> None:
        if not self.slots.is_held(slot):
            raise ValueError(f"slot {slot} is not held")

    # ------------------------------------------------------------------ growth

    def reserve(self, slots: Sequence[int], new_tokens: Sequence[int]) -> None:
        """Make room for ``new_tokens[i]`` more positions in ``slots[i]``.  Either every
        sequence gets its pages or none does and :class:`CacheCapacityError` is raised."""
        if len(set(slots)) != len(slots):
            raise ValueError(f"a slot appears twice in the batch: {list(slots)}")
        for group in self.kv_groups:
            extra = 0
            for slot, t in zip(slots, new_tokens):
                self._require_held(slot)
                extra += group.pages_needed(self.lengths[slot] + t) - len(group.slot_pages[slot])
            if extra > group.pages.free_count:
                total = sum(self.lengths[s] + t for s, t in zip(slots, new_tokens))
                raise CacheCapacityError(
                    f"KV cache capacity exceeded: the batch needs {extra} more pages of {PAGE_SIZE} tokens "
                    f"({total} tokens in {len(slots)} sequences), {group.pages.free_count} of "
                    f"{group.pages.count} pages are free (capacity {self.max_tokens} tokens)")
        for group in self.kv_groups:
            for slot, t in zip(slots, new_tokens):
                need = group.pages_needed(self.lengths[slot] + t) - len(group.slot_pages[slot])
                if need > 0:
                    group.slot_pages[slot].extend(group.pages.take_many(need))

    def advance(self, slots: Sequence[int], new_tokens: Sequence[int]) -> None:
        for slot, t in zip(slots, new_tokens):
            self.lengths[slot] += t

    # ------------------------------------------------------------------ views and figures

    def view(self, entry: int) -> CacheView:
        return self._views[entry]

    @property
    def storage_bytes(self) -> int:
        total = sum(g.pool.numel() * g.pool.element_size() for g in self.kv_groups)
        return total + sum(g.data.numel() * g.data.element_size() for g in self.state_groups)

    @property
    def tokens_held(self) -> int:
        """Tokens that live sequences hold, each rounded up to whole pages."""
        return sum(pages_for(self.lengths[s]) * PAGE_SIZE for s in range(self.max_seqs) if self.slots.is_held(s))

    def check(self) -> None:
        """Every slot and page is free or held exactly once; held pages belong to held slots."""
        self.slots.check()
        for group in self.kv_groups:
            group.pages.check()
            seen = set()
            for slot, pages in enumerate(group.slot_pages[:self.max_seqs]):
                if pages and not self.slots.is_held(slot):
                    raise AssertionError(f"free slot {slot} still holds pages")
                for page in pages:
                    if page in seen or not group.pages.is_held(page):
                        raise AssertionError(f"page {page} is held twice or not marked held")
                    seen.add(page)
            if len(seen) != group.pages.held_count:
                raise AssertionError("a held page belongs to no slot")
