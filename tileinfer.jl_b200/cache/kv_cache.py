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

The books (which slots are held, every sequence's length and pages, the pools' free lists) are kept by
the C++ host runtime (``csrc/host/cache_book.cpp``), which also writes new block-table entries to the
device and zeroes fresh pages with one kernel; this module allocates the storage and wraps the books.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..kernels import host
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
    extra: object = None                    # whatever a registered kind of its own hands to its mixer


# The kinds of storage a CacheRequest can name. A group class has
#   create(cache, index, request, layers) -> group   (classmethod; `layers` are the layers with this request)
#   views() -> [LayerCache]                           one per layer, in the order of `layers`
#   start(slot)                                       a sequence begins in `slot` (clear what the last one left)
#   paged                                             True only for storage in pages, which the books and the step planner handle
#   rolls_back                                        False if a sequence cannot be cut back to an earlier length
_GROUP_KINDS: Dict[str, type] = {}


def register_cache_kind(name: str):
    def deco(cls):
        cls.kind = name
        _GROUP_KINDS[name] = cls
        return cls
    return deco


def _stream(device) -> Optional[int]:
    if torch.device(device).type != "cuda":
        return None
    from ..kernels import library
    return library.current_stream()


class _Pages:
    """A paged group's pool of page numbers, as the books see it."""

    def __init__(self, group):
        self._g = group

    @property
    def free(self) -> int:
        return self._g._api.group_pages_free(self._g._book, self._g.book_index)

    @property
    def held(self) -> int:
        return self._g._api.group_pages_held(self._g._book, self._g.book_index)

    def is_held(self, page: int) -> bool:
        return bool(self._g._api.group_page_is_held(self._g._book, self._g.book_index, page))


@register_cache_kind("paged_kv")
class PagedGroup:
    paged, rolls_back = True, True

    @classmethod
    def create(cls, cache, index, request, layers):
        pages = cache.num_pages
        if request.window and cache.max_step_tokens:
            # Each sequence: the pages that its window touches, the release unit's slack and the
            # page that it writes to; plus the tokens of one step.
            per_seq = -(-(request.window - 1) // cache.page_size) + cache.release_granule + 1
            pages = min(pages, cache.max_seqs * per_seq + -(-cache.max_step_tokens // cache.page_size))
        max_pages_per_seq = -(-cache.max_seq_len // cache.page_size)
        bi = cache._api.cache_add_group(cache._book, pages, cache.page_size, request.window or 0, cache.release_granule,
                                        max_pages_per_seq)
        return cls(index, cache._book, bi, request, layers, pages, cache.page_size, cache.max_seqs, max_pages_per_seq,
                   cache.dtype, cache.device, cache.release_granule)

    def views(self):
        return [LayerCache(self.index, self.kind, self.page_size, self.k[j], self.v[j]) for j in range(len(self.layers))]

    def start(self, slot: int) -> None:
        pass                                   # fresh pages are zeroed as they are handed out

    def __init__(self, index, book, book_index, request: CacheRequest, layers: List[int], num_pages: int, page_size: int,
                 max_seqs: int, max_pages_per_seq: int, dtype, device, release_granule: int = 1):
        self.index, self.request, self.layers = index, request, layers
        self.page_size, self.num_pages = page_size, num_pages
        self.window = request.window or 0
        self.release_granule = max(1, release_granule)
        self.max_seqs, self.max_pages_per_seq = max_seqs, max_pages_per_seq
        self._api, self._book, self.book_index = host.api(), book, book_index      # book_index: among the paged groups
        shape = (len(layers), num_pages, request.kv_heads, page_size, request.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        self.device_table = torch.zeros((max_seqs, max_pages_per_seq), dtype=torch.int32, device=device)
        page_bytes = request.kv_heads * page_size * request.head_dim * self.v.element_size()
        self._api.cache_group_storage(book, book_index, self.device_table.data_ptr(), self.device_table.stride(0), self.v.data_ptr(),
                                      len(layers), num_pages * page_bytes, page_bytes, int(torch.device(device).type == "cuda"))
        # The host's copy of the block tables lives in the books; the step planner reads it there.
        raw = ctypes.cast(self._api.group_host_table(book, book_index), ctypes.POINTER(ctypes.c_int32))
        self.host_table = torch.from_numpy(np.ctypeslib.as_array(raw, shape=(max_seqs, max_pages_per_seq)))
        self.pages = _Pages(self)

    def table(self, slot: int) -> List[Optional[int]]:
        """The pages of a sequence by logical index; None where a page was given back behind the window."""
        buf = (ctypes.c_int * self.max_pages_per_seq)()
        n = self._api.group_table(self._book, self.book_index, slot, buf, self.max_pages_per_seq)
        return [None if buf[i] < 0 else buf[i] for i in range(n)]

    @property
    def tables(self) -> Dict[int, List[Optional[int]]]:
        out = {}
        for slot in range(self.max_seqs):
            t = self.table(slot)
            if t:
                out[slot] = t
        return out

    @property
    def first(self) -> Dict[int, int]:
        """Logical index of each sequence's first page that is still held (sequences that gave pages back only)."""
        firsts = {s: self._api.group_first(self._book, self.book_index, s) for s in range(self.max_seqs)}
        return {s: f for s, f in firsts.items() if f}

    def first_needed_page(self, length: int) -> int:
        """Logical index of the first page that a query at position ``length`` or later can read."""
        if not self.window:
            return 0
        key = max(0, length - self.window + 1)
        return key // self.page_size // self.release_granule * self.release_granule

    def peak_pages(self, growth: Sequence[Tuple[int, int]], chunk_tokens: Optional[int]) -> int:
        """Most pages beyond those held now that ``growth`` = [(slot, n)] needs at any time when it
        runs in token order in chunks of ``chunk_tokens`` and every chunk's end releases what fell out
        of the window."""
        return int(self._api.group_peak_pages(self._book, self.book_index, len(growth), host.ints(s for s, _ in growth),
                                              host.longs(n for _, n in growth), chunk_tokens or 0))

    def bytes_per_position(self) -> int:
        r = self.request
        return 2 * len(self.layers) * r.kv_heads * r.head_dim * self.k.element_size()


@register_cache_kind("state")
class StateGroup:
    paged, rolls_back = False, False

    @classmethod
    def create(cls, cache, index, request, layers):
        return cls(index, request, layers, cache.max_seqs, cache.dtype, cache.device)

    def __init__(self, index, request: CacheRequest, layers: List[int], max_seqs: int, dtype, device):
        self.index, self.request, self.layers = index, request, layers
        self.state = torch.zeros((len(layers), max_seqs) + tuple(request.shape), dtype=request.dtype or dtype, device=device)

    def views(self):
        return [LayerCache(self.index, self.kind, state=self.state[j]) for j in range(len(self.layers))]

    def start(self, slot: int) -> None:
        self.state[:, slot].zero_()


class _Slots:
    def __init__(self, cache):
        self._c = cache

    @property
    def held(self) -> int:
        return self._c._api.cache_slots_held(self._c._book)

    @property
    def free(self) -> int:
        return self._c.max_seqs - self.held

    def is_held(self, slot: int) -> bool:
        return bool(self._c._api.cache_slot_is_held(self._c._book, slot))


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
        self.release_granule = release_granule
        by_key: Dict[tuple, List[int]] = {}
        for i, r in enumerate(requests):
            if r is not None:
                by_key.setdefault(r.group_key(), []).append(i)
        kinds = {requests[layers[0]].kind for layers in by_key.values()}
        for kind in sorted(kinds):
            if kind not in _GROUP_KINDS:
                raise ValueError(f"unknown cache kind {kind!r} (registered: {', '.join(sorted(_GROUP_KINDS))})")
        self._api = host.api()
        self._book = self._api.cache_create(max_seqs, self.max_seq_len, int(any(not _GROUP_KINDS[k].rolls_back for k in kinds)))
        self.slots = _Slots(self)
        self.groups = []
        self._layer_view: Dict[int, LayerCache] = {}
        for key, layers in by_key.items():
            r = requests[layers[0]]
            g = _GROUP_KINDS[r.kind].create(self, len(self.groups), r, layers)
            for l, view in zip(layers, g.views()):
                self._layer_view[l] = view
            self.groups.append(g)
        for reader, source in (share or {}).items():
            self._layer_view[reader] = self._layer_view[source]
        self.paged_groups = [g for g in self.groups if g.paged]
        self.state_groups = [g for g in self.groups if not g.paged]
        self.windowed_groups = [g for g in self.paged_groups if g.window]

    def __del__(self):
        if getattr(self, "_book", None):
            self._api.cache_destroy(self._book)
            self._book = None

    @property
    def book(self):
        """The C++ books' handle (the step planner and the decode loop work on it directly)."""
        return self._book

    def _refused(self):
        raise ValueError(host.last_error())

    # ---- slots
    def alloc_slot(self) -> int:
        slot = self._api.cache_alloc_slot(self._book)
        if slot < 0:
            raise OutOfSlotsError(f"no free sequence slot (all {self.max_seqs} are held)")
        for g in self.groups:
            g.start(slot)
        return slot

    def free_slot(self, slot: int) -> None:
        if self._api.cache_free_slot(self._book, slot):
            self._refused()

    def length(self, slot: int) -> int:
        n = self._api.cache_length(self._book, slot)
        if n < 0:
            raise KeyError(f"sequence slot {slot} is not held")
        return int(n)

    @property
    def lengths(self) -> Dict[int, int]:
        """Length of every held sequence, by slot."""
        out = {}
        for slot in range(self.max_seqs):
            n = self._api.cache_length(self._book, slot)
            if n >= 0:
                out[slot] = int(n)
        return out

    # ---- pages
    def reserve(self, growth: Sequence[Tuple[int, int]], chunk_tokens: Optional[int] = None) -> None:
        """Make room for ``n`` more positions of each ``(slot, n)``. Either every sequence gets its
        pages or nothing changes (OutOfPagesError), as in src/kv/block_manager.jl:58-65. With
        ``chunk_tokens`` the caller runs the tokens in order in chunks of that many, calling ``prepare``
        before and ``advance`` after each: groups with a window then take their pages chunk by chunk."""
        needed, free = ctypes.c_longlong(), ctypes.c_longlong()
        rc = self._api.cache_reserve(self._book, len(growth), host.ints(s for s, _ in growth), host.longs(n for _, n in growth),
                                     chunk_tokens or 0, _stream(self.device), ctypes.byref(needed), ctypes.byref(free))
        if rc == 1:
            raise OutOfPagesError(needed.value, free.value)
        if rc:
            self._refused()

    def prepare(self, growth: Sequence[Tuple[int, int]]) -> None:
        """Before a chunk of a reserved step runs: the pages of this chunk for the groups that take
        them chunk by chunk (``reserve`` has checked that they are there)."""
        if self.windowed_groups and self._api.cache_prepare(self._book, len(growth), host.ints(s for s, _ in growth),
                                                            host.longs(n for _, n in growth), _stream(self.device)):
            self._refused()

    def advance(self, slot: int, n: int) -> None:
        """The step that wrote ``n`` more positions of ``slot`` has been enqueued."""
        if self._api.cache_advance(self._book, slot, n):
            self._refused()

    def truncate(self, slot: int, length: int) -> None:
        """Forget the positions after the first ``length`` (src/kv/block_manager.jl:74-81). Only paged
        storage can roll back; a state cannot."""
        if self._api.cache_truncate(self._book, slot, length):
            self._refused()

    def layer(self, index: int) -> LayerCache:
        return self._layer_view[index]

    def bytes_per_position(self) -> int:
        return sum(g.bytes_per_position() for g in self.paged_groups)

    def free_pages(self) -> int:
        return min((g.pages.free for g in self.paged_groups), default=0)
