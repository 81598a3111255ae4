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

A group with a window gives a sequence's pages back as they fall out of the window: after a
step that leaves a sequence at length L the next query sits at position L or later and sees
keys from L - window + 1 on, so the whole pages before that key return to the group's pool
(in steps of ``release_granule`` pages, the largest aligned unit in which a kernel walks the
keys). Its pool is therefore sized for ``max_seqs`` windows plus the tokens of one step, not
for ``max_tokens``; a long step is held chunk by chunk (``reserve`` checks the peak over the
chunks, ``prepare`` takes each chunk's pages).

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
                 max_pages_per_seq: int, dtype, device, release_granule: int = 1):
        self.index, self.request, self.layers = index, request, layers
        self.page_size, self.num_pages = page_size, num_pages
        self.window = request.window or 0
        self.release_granule = max(1, release_granule)
        self.first: Dict[int, int] = {}          # logical index of a sequence's first page that is still held
        shape = (len(layers), num_pages, request.kv_heads, page_size, request.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        self.pages = NumberPool(num_pages, "page")
        self.tables: Dict[int, List[int]] = {}
        self.max_pages_per_seq = max_pages_per_seq
        self._pin = torch.device(device).type == "cuda"
        self.host_table = torch.zeros((max_seqs, max_pages_per_seq), dtype=torch.int32)      # the host's copy, read by the step planner
        self.device_table = torch.zeros((max_seqs, max_pages_per_seq), dtype=torch.int32, device=device)

    def pages_needed(self, slot: int, new_length: int) -> int:
        have = len(self.tables.get(slot, ()))
        return max(0, -(-new_length // self.page_size) - have)

    def grow_many(self, growth: Sequence[Tuple[int, int]]) -> None:
        """Pages for each ``(slot, new length)`` (the caller has checked that the pool has them): the block
        tables' new entries go up in ONE copy and the new pages' values are zeroed by ONE kernel."""
        rows, cols, numbers = [], [], []
        for slot, new_length in growth:
            need = self.pages_needed(slot, new_length)
            if not need:
                continue
            table = self.tables.setdefault(slot, [])
            if len(table) + need > self.max_pages_per_seq:
                raise ValueError(f"a sequence of {new_length} positions needs more than {self.max_pages_per_seq} pages")
            new = self.pages.take_many(need)
            a = len(table)
            table.extend(new)
            self.host_table[slot, a:a + need] = torch.tensor(new, dtype=torch.int32)
            rows += [slot] * need
            cols += range(a, a + need)
            numbers += new
        if not numbers:
            return
        # The upload reads its source when the stream gets there, which may be after a slot has been freed
        # and handed to another sequence: it has a pinned buffer of its own (the allocator keeps it until the
        # copy has run), never the host table, which the next owner overwrites at once.
        packed = torch.tensor([rows, cols, numbers], dtype=torch.int64)
        packed = (packed.pin_memory() if self._pin else packed).to(self.device_table.device, non_blocking=True)
        self.device_table[packed[0], packed[1]] = packed[2].to(torch.int32)
        # A page's last user may have left anything in it. Keys beyond a sequence's length are masked by
        # selection, but their values take part in P V with weight 0, and 0 times a stale infinity or NaN
        # is NaN: values are zeroed when a page is taken.
        self.v.index_fill_(1, packed[2], 0)

    def grow(self, slot: int, new_length: int) -> None:
        self.grow_many([(slot, new_length)])

    def first_needed_page(self, length: int) -> int:
        """Logical index of the first page that a query at position ``length`` or later can read."""
        if not self.window:
            return 0
        key = max(0, length - self.window + 1)
        return key // self.page_size // self.release_granule * self.release_granule

    def release(self, slot: int, length: int) -> int:
        """Give back the pages that no query after ``length`` positions can see; returns how many."""
        table = self.tables.get(slot)
        if not self.window or not table:
            return 0
        a, b = self.first.get(slot, 0), min(self.first_needed_page(length), len(table))
        for i in range(a, b):
            self.pages.give(table[i])
            table[i] = None
        if b > a:
            self.first[slot] = b
        return max(0, b - a)

    def shrink(self, slot: int, new_length: int) -> None:
        table = self.tables.get(slot, [])
        keep = -(-new_length // self.page_size)
        if keep and self.first_needed_page(new_length) < self.first.get(slot, 0):
            raise ValueError(f"cannot roll back to {new_length} positions: the pages of its window were given back")
        for p in reversed(table[keep:]):
            if p is not None:
                self.pages.give(p)
        del table[keep:]
        if not table:
            self.tables.pop(slot, None)
            self.first.pop(slot, None)

    def peak_pages(self, growth, lengths: Dict[int, int], chunk_tokens: Optional[int]) -> int:
        """Most pages beyond those held now that ``growth`` = [(slot, n)] needs at any time when it
        runs in token order in chunks of ``chunk_tokens`` and every chunk's end releases what fell out
        of the window."""
        logical = {s: len(self.tables.get(s, ())) for s, _ in growth}
        first = {s: self.first.get(s, 0) for s, _ in growth}
        length = {s: lengths[s] for s, _ in growth}
        extra = peak = 0
        room = chunk_tokens or (1 << 62)
        touched = []
        for slot, n in growth:
            a = 0
            while a < n:
                take = min(room, n - a)
                length[slot] += take
                need = max(0, -(-length[slot] // self.page_size) - logical[slot])
                logical[slot] += need
                extra += need
                touched.append(slot)
                a += take
                room -= take
                if room == 0:
                    peak = max(peak, extra)
                    for s in touched:
                        b = min(self.first_needed_page(length[s]), logical[s])
                        extra -= max(0, b - first[s])
                        first[s] = max(first[s], b)
                    touched, room = [], chunk_tokens
        return max(peak, extra)

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
    each sequence rounded up to whole pages. ``max_step_tokens``: the most tokens that run between two
    calls of ``advance`` (it sizes the pools of groups with a window; None: sized like the others)."""

    def __init__(self, requests: Sequence[Optional[CacheRequest]], dtype: torch.dtype, device="cuda",
                 max_tokens: int = 4096, max_seqs: int = 8, page_size: int = DEFAULT_PAGE_SIZE,
                 max_seq_len: Optional[int] = None, share: Optional[Dict[int, int]] = None,
                 max_step_tokens: Optional[int] = None, release_granule: int = 2):
        if max_tokens < 1 or max_seqs < 1 or page_size < 1:
            raise ValueError("max_tokens, max_seqs and page_size must be positive")
        self.dtype, self.device = dtype, device
        self.page_size, self.max_seqs = page_size, max_seqs
        self.num_pages = -(-max_tokens // page_size)
        self.max_tokens = self.num_pages * page_size
        self.max_seq_len = min(max_seq_len or self.max_tokens, self.max_tokens)
        self.max_step_tokens = max_step_tokens
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
                pages = self.num_pages
                if r.window and max_step_tokens:
                    # Each sequence: the pages that its window touches, the release unit's slack and the
                    # page that it writes to; plus the tokens of one step.
                    per_seq = -(-(r.window - 1) // page_size) + release_granule + 1
                    pages = min(pages, max_seqs * per_seq + -(-max_step_tokens // page_size))
                g = PagedGroup(gi, r, layers, pages, page_size, max_seqs, max_pages_per_seq, dtype, device,
                               release_granule)
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
        self.windowed_groups = [g for g in self.paged_groups if g.window]

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
    def reserve(self, growth: Sequence[Tuple[int, int]], chunk_tokens: Optional[int] = None) -> None:
        """Make room for ``n`` more positions of each ``(slot, n)``. Either every sequence gets its
        pages or nothing changes (OutOfPagesError), as in src/kv/block_manager.jl:58-65. With
        ``chunk_tokens`` the caller runs the tokens in order in chunks of that many, calling ``prepare``
        before and ``advance`` after each: groups with a window then take their pages chunk by chunk."""
        for slot, n in growth:
            if not self.slots.is_held(slot):
                raise ValueError(f"sequence slot {slot} is not held")
            if self.lengths[slot] + n > self.max_seq_len:
                raise ValueError(f"sequence would reach {self.lengths[slot] + n} positions; the cache was sized for "
                                 f"sequences of at most {self.max_seq_len}")
        chunked = chunk_tokens is not None and sum(n for _, n in growth) > chunk_tokens
        for g in self.paged_groups:
            if g.window and chunked:
                need = g.peak_pages(growth, self.lengths, chunk_tokens)
            else:
                need = sum(g.pages_needed(slot, self.lengths[slot] + n) for slot, n in growth)
            if need > g.pages.free:
                raise OutOfPagesError(need, g.pages.free)
        for g in self.paged_groups:
            if not (g.window and chunked):
                g.grow_many([(slot, self.lengths[slot] + n) for slot, n in growth])

    def prepare(self, growth: Sequence[Tuple[int, int]]) -> None:
        """Before a chunk of a reserved step runs: the pages of this chunk for the groups that take
        them chunk by chunk (``reserve`` has checked that they are there)."""
        for g in self.windowed_groups:
            g.grow_many([(slot, self.lengths[slot] + n) for slot, n in growth])

    def advance(self, slot: int, n: int) -> None:
        """The step that wrote ``n`` more positions of ``slot`` has been enqueued."""
        self.lengths[slot] += n
        for g in self.windowed_groups:
            g.release(slot, self.lengths[slot])

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
