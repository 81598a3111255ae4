"""Allocators of the cache: pages of a pool and sequence slots.

Both hand out the lowest free number first and refuse to free what is not held, so a test
can tell that no slot or page is lost, held twice or freed twice. AntoineBut/TileInfer.jl's
BlockManager is the model for the page side (src/kv/block_manager.jl:39-100): pages come
out in increasing order, and a reservation that cannot be met changes nothing. The pools
themselves are C++ (``csrc/host/host_common.h``); this class is a pool on its own.
"""
from __future__ import annotations

from typing import Iterable, List

from ..kernels import host


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
        self._api = host.api()
        self._h = self._api.pool_create(count)

    def __del__(self):
        if getattr(self, "_h", None):
            self._api.pool_destroy(self._h)
            self._h = None

    @property
    def free(self) -> int:
        return self._api.pool_free(self._h)

    @property
    def held(self) -> int:
        return self._api.pool_held(self._h)

    def take(self) -> int:
        n = self._api.pool_take(self._h)
        if n < 0:
            raise OutOfSlotsError(f"no free {self.what} (all {self.count} are held)")
        return n

    def take_many(self, k: int) -> List[int]:
        if k > self.free:
            raise OutOfPagesError(k, self.free)
        return [self.take() for _ in range(k)]

    def give(self, n: int) -> None:
        if self._api.pool_give(self._h, n):
            raise ValueError(f"{self.what} {n} is not held (freed twice, or never allocated)")

    def give_many(self, ns: Iterable[int]) -> None:
        for n in ns:
            self.give(n)

    def is_held(self, n: int) -> bool:
        return bool(self._api.pool_is_held(self._h, n))
