"""The step's metadata, built on the host (csrc/host/step_planner.cpp through engine/step.py): positions, cache places, sequence ranges and
wanted rows of batches of unequal sequences, and the short path for one-token steps, which must write
exactly what the general one writes. Runs on the CPU (the planner only fills integer buffers)."""
import random

import numpy as np
import pytest
import torch

from tileinfer_b200.cache import Cache
from tileinfer_b200.engine.step import StepPlanner
from tileinfer_b200.kernels.fast import SplitKvPlan, split_tables
from tileinfer_b200.parts import CacheRequest


def make(page_size=4, max_seqs=5, max_tokens=200, window=None):
    cache = Cache([CacheRequest("paged_kv", kv_heads=2, head_dim=16, window=window)], torch.float32, "cpu",
                  max_tokens=max_tokens, max_seqs=max_seqs, page_size=page_size)
    return cache, StepPlanner(cache, 64, "cpu")


def place(cache, slot, position):
    g = cache.paged_groups[0]
    return int(g.host_table[slot, position // g.page_size]) * g.page_size + position % g.page_size


def test_a_batch_of_unequal_sequences():
    cache, planner = make()
    a, b, c = cache.alloc_slot(), cache.alloc_slot(), cache.alloc_slot()
    cache.reserve([(a, 6), (b, 1), (c, 9)])
    ctx = planner.plan([(a, [1, 2, 3, 4, 5, 6]), (b, [7]), (c, list(range(10, 19)))], [[0, 5], [], [8]])
    assert (ctx.n_tokens, ctx.n_seqs, ctx.n_want) == (16, 3, 3) and not ctx.is_decode
    assert ctx.token_ids.tolist() == [1, 2, 3, 4, 5, 6, 7] + list(range(10, 19))
    assert ctx.positions.tolist() == list(range(6)) + [0] + list(range(9))
    assert ctx.tok_slot.tolist() == [a] * 6 + [b] + [c] * 9
    assert ctx.cu_seqlens.tolist() == [0, 6, 7, 16] and ctx.kv_lens.tolist() == [6, 1, 9]
    assert ctx.want_idx.tolist() == [0, 5, 15]
    want = [place(cache, a, p) for p in range(6)] + [place(cache, b, 0)] + [place(cache, c, p) for p in range(9)]
    assert ctx.group(0).slot_mapping.tolist() == want and len(set(want)) == 16          # no two tokens share a place
    for s, n in ((a, 6), (b, 1), (c, 9)):
        cache.advance(s, n)
    # The next step continues where the sequences stand: one token each, the middle one gone.
    cache.free_slot(b)
    cache.reserve([(a, 1), (c, 1)])
    ctx = planner.plan([(a, [40]), (c, [41])], [[0], [0]])
    assert ctx.is_decode and ctx.positions.tolist() == [6, 9] and ctx.kv_lens.tolist() == [7, 10]
    assert ctx.group(0).slot_mapping.tolist() == [place(cache, a, 6), place(cache, c, 9)]
    with pytest.raises(ValueError, match="outside"):
        planner.plan([(a, [1])], [[1]])


def test_a_one_token_step_of_more_sequences_than_a_cut_step_has_tokens():
    """Steps of several tokens per sequence are cut at max_step_tokens, one-token steps never are: 40 sequences
    with a planner of 8 tokens a step go through both paths, and the general path refuses what it cannot hold
    instead of writing past its buffers."""
    cache = Cache([CacheRequest("paged_kv", kv_heads=2, head_dim=16)], torch.float32, "cpu", max_tokens=400, max_seqs=40, page_size=4)
    planner = StepPlanner(cache, 8, "cpu")
    slots = [cache.alloc_slot() for _ in range(40)]
    for i, s in enumerate(slots):
        cache.reserve([(s, 1 + i % 5)])
        cache.advance(s, 1 + i % 5)
    cache.reserve([(s, 1) for s in slots])
    short = planner.plan_decode(slots, list(range(40)))
    assert short.token_ids.tolist() == list(range(40)) and short.positions.tolist() == [1 + i % 5 for i in range(40)]
    assert short.kv_lens.tolist() == [2 + i % 5 for i in range(40)] and short.want_idx.tolist() == list(range(40))
    places = short.group(0).slot_mapping.tolist()
    assert places == [place(cache, s, 1 + i % 5) for i, s in enumerate(slots)] and len(set(places)) == 40
    o, _ = planner._layout(40, 40, 40)
    assert o["end"] <= planner.capacity
    first = planner.meta[:o["end"]].clone()
    with pytest.raises(ValueError, match="max_step_tokens"):
        planner.plan([(slots[0], list(range(9)))], [[0]])
    assert torch.equal(planner.meta[:o["end"]], first)


def test_the_short_path_for_one_token_steps_writes_what_the_general_one_writes():
    rng = random.Random(3)
    cache, planner = make(max_seqs=6, max_tokens=400)
    plan = SplitKvPlan(2, 4, 400)                                  # decode attention's work tables too
    planner.attach_plan(cache.paged_groups[0], plan)
    assert plan.splits(6) > 1
    slots = [cache.alloc_slot() for _ in range(6)]
    for s in slots:
        n = rng.randrange(1, 40)
        cache.reserve([(s, n)])
        cache.advance(s, n)
    for _ in range(30):
        live = rng.sample(slots, rng.randrange(1, 7))
        tokens = [rng.randrange(1000) for _ in live]
        cache.reserve([(s, 1) for s in live])
        general = planner.plan([(s, [t]) for s, t in zip(live, tokens)], [[0]] * len(live))
        words = general.n_tokens
        o, _ = planner._layout(words, words, words)
        first = planner.meta[:o["end"]].clone()
        planner.meta.zero_()
        short = planner.plan_decode(live, tokens)
        assert torch.equal(planner.meta[:o["end"]], first) and o["plan_words"][0] > 0
        work, seq = plan.tables(len(live), short.group(0).plan_table)
        assert short.group(0).plan is plan and work.numel() == 2 * len(live) * plan.splits(len(live)) and seq.numel() == len(live)
        assert short.is_decode and short.host_starts == general.host_starts and short.max_kv_len == general.max_kv_len
        for s in live:
            cache.advance(s, 1)


def test_decode_work_tables_cover_every_page_once():
    """Every sequence's parts are consecutive slots, there are as many as its entry says, none beyond the
    launch's B x splits, and long sequences get more of them."""
    rng = np.random.default_rng(0)
    for B, splits in ((1, 32), (3, 8), (8, 4), (5, 2)):
        for _ in range(20):
            lengths = rng.integers(1, 3000, size=B)
            work, seq = split_tables(lengths, splits, 64)
            assert work.shape == (B * splits, 2)
            used = 0
            for b in range(B):
                first, parts = int(seq[b]) >> 8, int(seq[b]) & 255
                assert first == used and 1 <= parts <= min(32, -(-int(lengths[b]) // 64))
                for i in range(parts):
                    w = int(work[first + i, 0])
                    assert (w >> 16, (w >> 8) & 255, w & 255) == (b, i, parts) and int(work[first + i, 1]) == int(lengths[b])
                used += parts
            assert used <= B * splits and all(int(w) == -1 for w in work[used:, 0])
            order = np.argsort(lengths)
            parts_of = (seq & 255)[order]
            assert all(parts_of[i] <= parts_of[i + 1] for i in range(B - 1))           # more keys, no fewer parts


def test_every_legal_step_fits_the_metadata_buffers():
    """For random engine sizes (with and without the decode attention's tables, one or two cache groups): the layout of
    every step the engine may ask for (up to max_step_tokens tokens over up to max_seqs sequences, every token wanted;
    one token for each of up to max_seqs sequences) ends inside the planner's buffers."""
    rng = random.Random(11)
    for _ in range(40):
        max_seqs = rng.choice([1, 2, 7, 33, 64, 200])
        max_step = rng.choice([1, 5, 31, 32, 33, 500, 4096])
        requests = [CacheRequest("paged_kv", kv_heads=2, head_dim=16)]
        if rng.random() < 0.4:
            requests.append(CacheRequest("paged_kv", kv_heads=1, head_dim=32, window=24))
        cache = Cache(requests, torch.float32, "cpu", max_tokens=64 * max_seqs, max_seqs=max_seqs, page_size=rng.choice([4, 16, 64]))
        planner = StepPlanner(cache, max_step, "cpu")
        if rng.random() < 0.7:
            planner.attach_plan(cache.paged_groups[0], SplitKvPlan(2, cache.page_size, cache.max_tokens))
        cases = [(b, b, b) for b in {1, max_seqs, max(1, max_seqs // 2)}]
        cases += [(max_step, min(max_step, max_seqs), max_step), (max_step, 1, max_step), (max_step, min(max_step, max_seqs), 0)]
        for n, B, nw in cases:
            o, _ = planner._layout(n, B, nw)
            assert o["end"] <= planner.capacity, (max_seqs, max_step, n, B, nw, o["end"], planner.capacity)
