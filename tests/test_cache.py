"""The cache's host side: no slot or page lost, held twice or freed twice; failed reservations
change nothing (the reference's test/kv/block_manager.jl:1-29 is the model for the page side)."""
import random

import pytest
import torch

from tileinfer_b200.cache import Cache, NumberPool, OutOfPagesError, OutOfSlotsError
from tileinfer_b200.parts import CacheRequest


def kv(heads=2, dim=16, window=None):
    return CacheRequest("paged_kv", kv_heads=heads, head_dim=dim, window=window)


def make(requests=None, **kw):
    kw.setdefault("max_tokens", 8 * 4)
    kw.setdefault("max_seqs", 3)
    kw.setdefault("page_size", 4)
    return Cache(requests or [kv(), kv()], torch.float32, "cpu", **kw)


def test_number_pool_hands_out_lowest_first_and_refuses_double_free():
    p = NumberPool(3, "slot")
    assert [p.take(), p.take(), p.take()] == [0, 1, 2]
    with pytest.raises(OutOfSlotsError):
        p.take()
    p.give(1)
    with pytest.raises(ValueError, match="not held"):
        p.give(1)
    assert p.take() == 1 and p.free == 0 and p.held == 3


def test_pages_follow_lengths_and_come_back():
    c = make()
    g = c.paged_groups[0]
    a, b = c.alloc_slot(), c.alloc_slot()
    c.reserve([(a, 5), (b, 1)])
    assert g.tables[a] == [0, 1] and g.tables[b] == [2] and g.pages.free == 5
    c.advance(a, 5); c.advance(b, 1)
    c.reserve([(a, 3)])                      # 8 positions: still two pages
    assert g.tables[a] == [0, 1]
    c.advance(a, 3)
    c.reserve([(a, 1)])
    assert g.tables[a] == [0, 1, 3]
    assert g.host_table[a, :3].tolist() == [0, 1, 3] and g.device_table[a, :3].tolist() == [0, 1, 3]
    c.free_slot(a)
    assert g.pages.free == 7 and a not in g.tables
    with pytest.raises(ValueError, match="not held"):
        c.free_slot(a)
    assert c.alloc_slot() == a               # the slot is used again
    c.reserve([(a, 9)])
    assert g.tables[a] == [0, 1, 3]          # and so are its pages, lowest first


def test_failed_reservation_changes_nothing():
    c = make()
    a, b = c.alloc_slot(), c.alloc_slot()
    c.reserve([(a, 20)]); c.advance(a, 20)   # 5 of 8 pages
    g = c.paged_groups[0]
    before = (dict(g.tables), g.pages.free)
    with pytest.raises(OutOfPagesError) as e:
        c.reserve([(a, 4), (b, 12)])         # needs 1 + 3 pages, 3 free
    assert (e.value.needed, e.value.free) == (4, 3)
    assert (dict(g.tables), g.pages.free) == before
    with pytest.raises(ValueError, match="not held"):
        c.reserve([(2, 1)])


def test_sequence_length_limit_and_slot_limit():
    c = make(max_seq_len=10)
    s = c.alloc_slot()
    with pytest.raises(ValueError, match="at most 10"):
        c.reserve([(s, 11)])
    c.alloc_slot(); c.alloc_slot()
    with pytest.raises(OutOfSlotsError):
        c.alloc_slot()


def test_truncate_returns_pages():
    c = make()
    s = c.alloc_slot()
    c.reserve([(s, 14)]); c.advance(s, 14)
    g = c.paged_groups[0]
    assert len(g.tables[s]) == 4
    c.truncate(s, 5)
    assert g.tables[s] == [0, 1] and c.length(s) == 5 and g.pages.free == 6
    with pytest.raises(ValueError):
        c.truncate(s, 6)


def test_groups_by_need_have_their_own_storage():
    reqs = [kv(2, 16), kv(2, 16, window=8), kv(2, 16), CacheRequest("state", shape=(3, 5)), None]
    c = Cache(reqs, torch.float32, "cpu", max_tokens=32, max_seqs=2, page_size=4, share={4: 0})
    assert len(c.groups) == 3
    full, windowed, state = c.groups
    assert full.layers == [0, 2] and windowed.layers == [1] and state.layers == [3]
    assert full.k.shape == (2, 8, 2, 4, 16) and state.state.shape == (1, 2, 3, 5)
    assert c.layer(0).k.data_ptr() != c.layer(2).k.data_ptr()
    assert c.layer(4).k.data_ptr() == c.layer(0).k.data_ptr()          # layer 4 reads layer 0's keys
    assert c.layer(1).group_index == 1 and c.layer(3).kind == "state"
    s = c.alloc_slot()
    state.state[0, s] = 7.0
    c.free_slot(s)
    assert c.alloc_slot() == s and float(state.state[0, s].abs().sum()) == 0.0   # zeroed for its next user
    with pytest.raises(ValueError, match="roll back"):
        c.reserve([(s, 4)]); c.advance(s, 4); c.truncate(s, 2)


def test_a_third_kind_of_storage_is_registered_not_edited_in():
    """A kind of per-sequence storage defined HERE (a pair of tensors per layer and slot, marked as started with -1,
    able to roll back) is registered, built next to a paged group, started with every new sequence and handed to
    its layers; an unregistered kind is refused by name."""
    from tileinfer_b200.cache import LayerCache, register_cache_kind

    @register_cache_kind("toy_pair")
    class PairGroup:
        paged, rolls_back = False, True

        @classmethod
        def create(cls, cache, index, request, layers):
            g = cls()
            g.index, g.request, g.layers = index, request, layers
            g.a = torch.zeros((len(layers), cache.max_seqs) + tuple(request.shape))
            g.b = torch.zeros((len(layers), cache.max_seqs), dtype=torch.int64)
            g.started = []
            return g

        def views(self):
            return [LayerCache(self.index, self.kind, extra=(self.a[j], self.b[j])) for j in range(len(self.layers))]

        def start(self, slot):
            self.a[:, slot] = -1.0
            self.b[:, slot] = 0
            self.started.append(slot)

    reqs = [kv(), CacheRequest("toy_pair", shape=(3,)), kv(), CacheRequest("toy_pair", shape=(3,))]
    c = Cache(reqs, torch.float32, "cpu", max_tokens=32, max_seqs=2, page_size=4)
    paged, pair = c.groups
    assert paged.layers == [0, 2] and pair.layers == [1, 3] and pair.kind == "toy_pair"
    assert c.paged_groups == [paged] and c.layer(3).kind == "toy_pair"
    a, b = c.layer(3).extra
    assert a.data_ptr() == pair.a[1].data_ptr() and b.shape == (2,)
    s = c.alloc_slot()
    assert pair.started == [s] and float(a[s].sum()) == -3.0
    c.reserve([(s, 6)]); c.advance(s, 6); c.truncate(s, 2)                 # this kind rolls back: the books allow it
    assert c.length(s) == 2
    c.free_slot(s)
    assert c.alloc_slot() == s and pair.started == [s, s]
    with pytest.raises(ValueError, match="unknown cache kind 'ring'.*toy_pair"):
        Cache([kv(), CacheRequest("ring")], torch.float32, "cpu", max_tokens=32, max_seqs=2, page_size=4)


def test_random_traffic_keeps_the_books_straight():
    rng = random.Random(0)
    c = make(max_tokens=64 * 4, max_seqs=6)
    g = c.paged_groups[0]
    live = {}
    for _ in range(2000):
        op = rng.random()
        if op < 0.25 and len(live) < 6:
            live[c.alloc_slot()] = 0
        elif op < 0.45 and live:
            s = rng.choice(list(live)); c.free_slot(s); del live[s]
        elif live:
            s = rng.choice(list(live)); n = rng.randint(1, 9)
            try:
                c.reserve([(s, n)]); c.advance(s, n); live[s] += n
            except OutOfPagesError:
                pass
        held = [p for t in g.tables.values() for p in t]
        assert len(held) == len(set(held)) == g.pages.held            # no page held twice
        assert g.pages.held + g.pages.free == g.num_pages            # none lost
        assert all(len(g.tables.get(s, [])) == -(-n // 4) for s, n in live.items())
        assert c.slots.held == len(live)


def test_a_windowed_group_gives_pages_back_as_they_fall_out_of_the_window():
    """Window 10, pages of 4, release unit 2 pages: after L positions the next query sees keys from
    L - 9 on, so pages before floor((L - 9) / 4) rounded down to an even index are free again."""
    c = Cache([kv(), kv(window=10)], torch.float32, "cpu", max_tokens=64, max_seqs=2, page_size=4, release_granule=2)
    full, win = c.paged_groups
    s = c.alloc_slot()
    c.reserve([(s, 13)]); c.advance(s, 13)
    assert win.tables[s] == [0, 1, 2, 3] and win.first.get(s, 0) == 0          # key 4 is still seen: page 1, unit 0
    c.reserve([(s, 4)]); c.advance(s, 4)                                      # L = 17: first key 8, page 2
    assert win.tables[s] == [None, None, 2, 3, 4] and win.first[s] == 2 and win.pages.held == 3
    assert not win.pages.is_held(0) and not win.pages.is_held(1)              # pages 0 and 1 are free again
    assert full.tables[s] == [0, 1, 2, 3, 4]                                  # the other group keeps everything
    for _ in range(30):
        c.reserve([(s, 1)]); c.advance(s, 1)
        held = [p for p in win.tables[s] if p is not None]
        assert len(held) == win.pages.held <= 5 and len(set(held)) == len(held)
        assert win.first[s] == (c.length(s) - 9) // 4 // 2 * 2
        # every key that the next query sees lies on a held page
        assert all(win.tables[s][k // 4] is not None for k in range(c.length(s) - 9, c.length(s)))
    with pytest.raises(ValueError, match="roll back"):
        c.truncate(s, c.length(s) - 8)
    c.truncate(s, c.length(s) - 1)                                            # within the held pages: fine
    c.free_slot(s)
    assert win.pages.held == 0 and full.pages.held == 0 and win.first == {} and win.tables == {}


def test_a_windowed_pool_is_sized_for_windows_and_one_step_and_long_steps_run_in_chunks():
    c = Cache([kv(window=10)], torch.float32, "cpu", max_tokens=400, max_seqs=2, page_size=4, max_step_tokens=16,
              release_granule=2)
    (win,) = c.paged_groups
    assert win.num_pages == 2 * (3 + 2 + 1) + 4 < c.num_pages
    a, b = c.alloc_slot(), c.alloc_slot()
    growth = [(a, 150), (b, 90)]
    with pytest.raises(OutOfPagesError):
        c.reserve(growth)                                                     # whole, it does not fit
    assert win.pages.held == 0
    c.reserve(growth, chunk_tokens=16)                                        # chunk by chunk it does
    assert win.pages.held == 0
    # run the chunks as the engine does: tokens in order, 16 at a time
    peak, room, chunk = 0, 16, []
    def run(chunk):
        nonlocal peak
        c.prepare(chunk)
        peak = max(peak, win.pages.held)
        for s, n in chunk:
            c.advance(s, n)
    for s, n in growth:
        done = 0
        while done < n:
            take = min(room, n - done)
            chunk.append((s, take)); done += take; room -= take
            if room == 0:
                run(chunk); chunk, room = [], 16
    if chunk:
        run(chunk)
    assert c.length(a) == 150 and c.length(b) == 90 and peak <= win.num_pages
    # decoding on from there stays within the pool for ever
    for _ in range(100):
        c.reserve([(a, 1), (b, 1)]); c.advance(a, 1); c.advance(b, 1)
    assert win.pages.held <= 2 * 5
    c.free_slot(a); c.free_slot(b)
    assert win.pages.held == 0 and win.pages.free == win.num_pages


def test_the_peak_of_a_chunked_step_is_what_running_it_takes():
    rng = random.Random(1)
    for _ in range(50):
        window, chunk = rng.randint(1, 40), rng.randint(1, 50)
        c = Cache([kv(window=window)], torch.float32, "cpu", max_tokens=4000, max_seqs=3, page_size=4, release_granule=2)
        (win,) = c.paged_groups
        slots = [c.alloc_slot() for _ in range(3)]
        for s in slots:                                                       # some history first
            n = rng.randint(0, 60)
            if n:
                c.reserve([(s, n)]); c.advance(s, n)
        growth = [(s, rng.randint(1, 120)) for s in slots]
        before = win.pages.held
        predicted = win.peak_pages(growth, chunk)
        c.reserve(growth, chunk_tokens=chunk)
        peak, room, cur = before, chunk, []
        for s, n in growth:
            done = 0
            while done < n:
                take = min(room, n - done)
                cur.append((s, take)); done += take; room -= take
                if room == 0:
                    c.prepare(cur); peak = max(peak, win.pages.held)
                    for x, m in cur:
                        c.advance(x, m)
                    cur, room = [], chunk
        if cur:
            c.prepare(cur); peak = max(peak, win.pages.held)
            for x, m in cur:
                c.advance(x, m)
        assert peak - before == predicted
