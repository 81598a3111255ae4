"""Host-side allocators of the cache: pages of a pool and sequence slots.

Both hand out the lowest free number first and refuse to free what is not held, so a test
can tell that no slot or page is lost, held twice or freed twice. AntoineBut/TileInfer.jl's
BlockManager is the model for the page side (src/kv/block_manager.jl:39-100): pages come
out in increasing order, and a reservation that cannot be met changes nothing.
"""
from __future__ import annotations

import heapq
from typing import Iterable, List


class OutOfPagesError(RuntimeError):
    """The pool has fewer free pages than a step needs (src/kv/block_manager.jl:26-32)."""

    def __init__(self, needed: int, free: int):
        self.needed, self.free = needed, free
        super().__init__(f"KV cache full: need {needed} more pages, {free} free")


class OutOfSlotsError(RuntimeError):
    pass


class NumberPool:
    """Numbers 0..count-1; ``take`` gives the smallest free one, ``give`` returns one."""

    def __init__(self, count: int, what: str):
        self.count, self.what = count, what
        self._free = list(range(count))
        heapq.heapify(self._free)
        self._held = set()

    @property
    def free(self) -> int:
        return len(self._free)

    @property
    def held(self) -> int:
        return len(self._held)

    def take(self) -> int:
        if not self._free:
            raise OutOfSlotsError(f"no free {self.what} (all {self.count} are held)")
        n = heapq.heappop(self._free)
        self._held.add(n)
        return n

    def take_many(self, k: int) -> List[int]:
        if k > len(self._free):
            raise OutOfPagesError(k, len(self._free))
        return [self.take() for _ in range(k)]

    def give(self, n: int) -> None:
        if n not in self._held:
            raise ValueError(f"{self.what} {n} is not held (freed twice, or never allocated)")
        self._held.remove(n)
        heapq.heappush(self._free, n)

    def give_many(self, ns: Iterable[int]) -> None:
        for n in ns:
            self.give(n)

    def is_held(self, n: int) -> bool:
        return n in self._held
