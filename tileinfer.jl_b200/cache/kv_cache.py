"""The cache: a slot for each sequence of a batch, storage for each layer, grouped by need.

Every layer's mixer says what it needs per sequence (``CacheRequest``): keys and values of
all positions, of a window of them, or a state of fixed size. Layers with the same request
form a *group* with storage of its own: a paged group has one K and one V pool
``[layers, pages, kv_heads, page_size, head_dim]`` (a page of one head is a dense
``[page_size, head_dim]`` tile, as in AntoineBut/TileInfer.jl src/kv/paged_cache.jl:1-4,
18-36), its own page allocator and its own block table per sequence; a state group has one
tensor ``[layers, slots, *shape]`` that is zeroed when a slot is handed out. A sequence
holds one slot from its first step until it is freed; its pages and its slot then go back
and are used again.

The reference has one group, one sequence per step and a block table per ``Sequence``
object (src/kv/block_manager.jl:13-16); slots, groups and the per-sequence state are this
library's own.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..parts.base import CacheRequest
from .allocator import NumberPool, OutOfPagesError, OutOfSlotsError

DEFAULT_PAGE_SIZE = 64      # positions per page (src/kv/paged_cache.jl:7)


@dataclass
class LayerCache:
    """What one layer's mixer sees of the cache."""
    group_index: int
    kind: str
    page_size: int = 0
    k: Optional[torch.Tensor] = None        # [pages, kv_heads, page_size, head_dim]
    v: Optional[torch.Tensor] = None
    state: Optional[torch.Tensor] = None    # [slots, *shape]


class PagedGroup:
    kind = "paged_kv"

    def __init__(self, index, request: CacheRequest, layers: List[int], num_pages: int, page_size: int, max_seqs: int,
                 max_pages_per_seq: int, dtype, device):
        self.index, self.request, self.layers = index, request, layers
        self.page_size, self.num_pages = page_size, num_pages
        shape = (len(layers), num_pages, request.kv_heads, page_size, request.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        self.pages = NumberPool(num_pages, "page")
        self.tables: Dict[int, List[int]] = {}
        self.max_pages_per_seq = max_pages_per_seq
        pin = torch.device(device).type == "cuda"
        self.host_table = torch.zeros((max_seqs, max_pages_per_seq), dtype=torch.int32, pin_memory=pin)
        self.device_table = torch.zeros((max_seqs, max_pages_per_seq), dtype=torch.int32, device=device)

    def pages_needed(self, slot: int, new_length: int) -> int:
        have = len(self.tables.get(slot, ()))
        return max(0, -(-new_length // self.page_size) - have)

    def grow(self, slot: int, new_length: int) -> None:
        need = self.pages_needed(slot, new_length)
        if not need:
            return
        table = self.tables.setdefault(slot, [])
        if len(table) + need > self.max_pages_per_seq:
            raise ValueError(f"a sequence of {new_length} positions needs more than {self.max_pages_per_seq} pages")
        new = self.pages.take_many(need)
        a = len(table)
        table.extend(new)
        self.host_table[slot, a:a + need] = torch.tensor(new, dtype=torch.int32)
        self.device_table[slot, a:a + need].copy_(self.host_table[slot, a:a + need], non_blocking=True)

    def shrink(self, slot: int, new_length: int) -> None:
        table = self.tables.get(slot, [])
        keep = -(-new_length // self.page_size)
        for p in reversed(table[keep:]):
            self.pages.give(p)
        del table[keep:]
        if not table:
            self.tables.pop(slot, None)

    def bytes_per_position(self) -> int:
        r = self.request
        return 2 * len(self.layers) * r.kv_heads * r.head_dim * self.k.element_size()


class StateGroup:
    kind = "state"

    def __init__(self, index, request: CacheRequest, layers: List[int], max_seqs: int, dtype, device):
        self.index, self.request, self.layers = index, request, layers
        self.state = torch.zeros((len(layers), max_seqs) + tuple(request.shape), dtype=request.dtype or dtype, device=device)


class Cache:
    """``requests[i]`` is layer i's CacheRequest (None: the layer keeps nothing; it may read another
    layer's storage, see ``share``). ``max_tokens`` is the most positions live sequences hold together,
    each sequence rounded up to whole pages."""

    def __init__(self, requests: Sequence[Optional[CacheRequest]], dtype: torch.dtype, device="cuda",
                 max_tokens: int = 4096, max_seqs: int = 8, page_size: int = DEFAULT_PAGE_SIZE,
                 max_seq_len: Optional[int] = None, share: Optional[Dict[int, int]] = None):
        if max_tokens < 1 or max_seqs < 1 or page_size < 1:
            raise ValueError("max_tokens, max_seqs and page_size must be positive")
        self.dtype, self.device = dtype, device
        self.page_size, self.max_seqs = page_size, max_seqs
        self.num_pages = -(-max_tokens // page_size)
        self.max_tokens = self.num_pages * page_size
        self.max_seq_len = min(max_seq_len or self.max_tokens, self.max_tokens)
        max_pages_per_seq = -(-self.max_seq_len // page_size)
        self.slots = NumberPool(max_seqs, "sequence slot")
        self.lengths: Dict[int, int] = {}
        by_key: Dict[tuple, List[int]] = {}
        for i, r in enumerate(requests):
            if r is not None:
                by_key.setdefault(r.group_key(), []).append(i)
        self.groups = []
        self._layer_view: Dict[int, LayerCache] = {}
        for key, layers in by_key.items():
            r = requests[layers[0]]
            gi = len(self.groups)
            if r.kind == "paged_kv":
                g = PagedGroup(gi, r, layers, self.num_pages, page_size, max_seqs, max_pages_per_seq, dtype, device)
                for j, l in enumerate(layers):
                    self._layer_view[l] = LayerCache(gi, "paged_kv", page_size, g.k[j], g.v[j])
            elif r.kind == "state":
                g = StateGroup(gi, r, layers, max_seqs, dtype, device)
                for j, l in enumerate(layers):
                    self._layer_view[l] = LayerCache(gi, "state", state=g.state[j])
            else:
                raise ValueError(f"unknown cache kind {r.kind}")
            self.groups.append(g)
        for reader, source in (share or {}).items():
            self._layer_view[reader] = self._layer_view[source]
        self.paged_groups = [g for g in self.groups if g.kind == "paged_kv"]
        self.state_groups = [g for g in self.groups if g.kind == "state"]

    # ---- slots
    def alloc_slot(self) -> int:
        slot = self.slots.take()
        self.lengths[slot] = 0
        for g in self.state_groups:
            g.state[:, slot].zero_()
        return slot

    def free_slot(self, slot: int) -> None:
        if not self.slots.is_held(slot):
            raise ValueError(f"sequence slot {slot} is not held (freed twice, or never allocated)")
        for g in self.paged_groups:
            g.shrink(slot, 0)
        del self.lengths[slot]
        self.slots.give(slot)

    def length(self, slot: int) -> int:
        return self.lengths[slot]

    # ---- pages
    def reserve(self, growth: Sequence[Tuple[int, int]]) -> None:
        """Make room for ``n`` more positions of each ``(slot, n)``. Either every sequence gets its
        pages or nothing changes (OutOfPagesError), as in src/kv/block_manager.jl:58-65."""
        for slot, n in growth:
            if not self.slots.is_held(slot):
                raise ValueError(f"sequence slot {slot} is not held")
            if self.lengths[slot] + n > self.max_seq_len:
                raise ValueError(f"sequence would reach {self.lengths[slot] + n} positions; the cache was sized for "
                                 f"sequences of at most {self.max_seq_len}")
        for g in self.paged_groups:
            need = sum(g.pages_needed(slot, self.lengths[slot] + n) for slot, n in growth)
            if need > g.pages.free:
                raise OutOfPagesError(need, g.pages.free)
        for g in self.paged_groups:
            for slot, n in growth:
                g.grow(slot, self.lengths[slot] + n)

    def advance(self, slot: int, n: int) -> None:
        self.lengths[slot] += n

    def truncate(self, slot: int, length: int) -> None:
        """Forget the positions after the first ``length`` (src/kv/block_manager.jl:74-81). Only paged
        storage can roll back; a state cannot."""
        if not 0 <= length <= self.lengths[slot]:
            raise ValueError(f"cannot truncate a sequence of length {self.lengths[slot]} to {length}")
        if self.state_groups and length != self.lengths[slot]:
            raise ValueError("layers with a per-sequence state cannot roll back")
        for g in self.paged_groups:
            g.shrink(slot, length)
        self.lengths[slot] = length

    def layer(self, index: int) -> LayerCache:
        return self._layer_view[index]

    def bytes_per_position(self) -> int:
        return sum(g.bytes_per_position() for g in self.paged_groups)

    def free_pages(self) -> int:
        return min((g.pages.free for g in self.paged_groups), default=0)
