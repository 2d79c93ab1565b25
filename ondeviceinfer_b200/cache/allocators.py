"""Host-side bookkeeping: which slots and which pages are free.

Both allocators hand out small integers from a free list and refuse misuse loudly: an
index is never handed out twice, never returned twice, never returned unless it was
handed out.  ``check()`` verifies that every index is either free or held, exactly once.
"""

from __future__ import annotations

from typing import List


class CacheCapacityError(RuntimeError):
    """No slot or page is left."""


class IndexAllocator:
    def __init__(self, count: int, what: str) -> None:
        if count < 0:
            raise ValueError(f"number of {what}s must not be negative")
        self.count, self.what = count, what
        self._free: List[int] = list(range(count - 1, -1, -1))  # pop() hands out 0 first
        self._held = [False] * count

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held_count(self) -> int:
        return self.count - len(self._free)

    def take(self) -> int:
        if not self._free:
            raise CacheCapacityError(f"no free {self.what}: all {self.count} are held")
        index = self._free.pop()
        self._held[index] = True
        return index

    def take_many(self, n: int) -> List[int]:
        if n > len(self._free):
            raise CacheCapacityError(
                f"KV cache capacity exceeded: {n} more {self.what}s requested, {len(self._free)} of {self.count} free")
        return [self.take() for _ in range(n)]

    def give_back(self, index: int) -> None:
        if not 0 <= index < self.count:
            raise ValueError(f"{self.what} {index} does not exist (0..{self.count - 1})")
        if not self._held[index]:
            raise ValueError(f"{self.what} {index} is not held (freed twice, or never allocated)")
        self._held[index] = False
        self._free.append(index)

    def is_held(self, index: int) -> bool:
        return 0 <= index < self.count and self._held[index]

    def check(self) -> None:
        free = set(self._free)
        if len(free) != len(self._free):
            raise AssertionError(f"a {self.what} is in the free list twice")
        for index in range(self.count):
            if self._held[index] == (index in free):
                raise AssertionError(f"{self.what} {index} is {'both held and free' if self._held[index] else 'lost'}")
