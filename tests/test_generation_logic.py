"""Decisions of the generation loop that need no device: batching and when a sequence ends
(the reference's loop: src/engine/generate.jl:43-56)."""
import pytest

from tileinfer_b200.engine.generate import finished, plan_batches
from tileinfer_b200.sampling import SamplingParams, mix32, sequence_seed


def test_batches_respect_slots_and_pages():
    p = plan_batches([5, 9, 13, 70, 1], max_new_tokens=8, max_seqs=2, max_tokens=1024, page_size=64, max_context=512)
    assert p.batches == [[0, 1], [2, 3], [4]]
    p = plan_batches([60, 60, 60], max_new_tokens=8, max_seqs=8, max_tokens=256, page_size=64, max_context=512)
    assert p.batches == [[0, 1], [2]]            # 68 tokens round up to 128 each
    with pytest.raises(ValueError, match="max context"):
        plan_batches([510], 8, 2, 1024, 64, 512)
    with pytest.raises(ValueError, match="cache holds"):
        plan_batches([100], 100, 2, 128, 64, 512)
    with pytest.raises(ValueError, match="no tokens"):
        plan_batches([3, 0], 4, 2, 1024, 64, 512)


def test_when_a_sequence_ends():
    assert finished(7, 0, 10, {7}) == "stop"
    assert finished(3, 0, 10, {7}) == "go"
    assert finished(3, 9, 10, {7}) == "last"
    assert finished(7, 9, 10, {7}) == "stop"     # a stop token is never emitted, even as the last one
    assert finished(3, 0, 1, set()) == "last"


def test_sampling_params_are_validated():
    assert SamplingParams().greedy and not SamplingParams(temperature=0.8).greedy
    for bad in (dict(temperature=-1), dict(top_k=-1), dict(top_p=0.0), dict(top_p=1.5)):
        with pytest.raises(ValueError):
            SamplingParams(**bad)


def test_mix32_is_lowbias32_and_sequence_seeds_differ():
    def lowbias32(x):                                   # src/engine/sampler.jl:34-38, written out step by step
        x ^= x >> 16
        x = x * 0x7FEB352D % 2 ** 32
        x ^= x >> 15
        x = x * 0x846CA68B % 2 ** 32
        return x ^ (x >> 16)
    assert mix32(0) == 0
    for x in (1, 2, 0x12345678, 0xFFFFFFFF, 0x80000000, 12345):
        assert mix32(x) == lowbias32(x) and 0 <= mix32(x) < 2 ** 32
    assert len({mix32(x) for x in range(5000)}) == 5000          # a bijection has no collisions
    # The uniform numbers built on it, with the reference's own checks (test/engine/sampler.jl:68-76).
    import plain_apertus as plain
    u = [plain.sampling_uniform(seed, c) for seed in range(1, 21) for c in range(1000)]
    assert all(0 <= x < 1 for x in u) and abs(sum(u) / len(u) - 0.5) < 0.01
    counts = [sum(1 for x in u if (b - 1) / 10 <= x < b / 10) for b in range(1, 11)]
    assert all(abs(c - 2000) < 200 for c in counts)
    assert len(set(u[:1000])) == 1000 and plain.sampling_uniform(1, 0) != plain.sampling_uniform(2, 0)
    seeds = {sequence_seed(5, i) for i in range(100)}
    assert len(seeds) == 100 and sequence_seed(5, 3) != sequence_seed(6, 3)


def test_decode_work_slots_are_shared_out_by_length():
    """Every sequence gets at least one part and at most 32 and not more than it has pages; the parts of
    all sequences fit the slots; a sequence's slots are consecutive and numbered; equal lengths give
    every sequence the same number of parts; a long sequence among short ones gets most of them."""
    import numpy as np
    from tileinfer_b200.kernels.fast import split_tables
    rng = np.random.default_rng(0)
    for B, splits in ((1, 32), (3, 9), (8, 4), (8, 1), (37, 8), (64, 4)):
        for lengths in (np.full(B, 1023), rng.integers(1, 40000, B), np.array([1] * (B - 1) + [30000])):
            work, seq = split_tables(lengths.astype(np.int64), splits, 64)
            T = B * splits
            assert work.shape == (T, 2) and len(seq) == B
            first, parts = seq >> 8, seq & 255
            pages = -(-lengths // 64)
            assert (parts >= 1).all() and (parts <= 32).all() and (parts <= np.maximum(pages, 1)).all()
            assert int(parts.sum()) <= T and (first == np.cumsum(parts) - parts).all()
            for b in range(B):
                for s in range(int(parts[b])):
                    assert work[first[b] + s].tolist() == [(b << 16) | (s << 8) | int(parts[b]), int(lengths[b])]
            assert (work[int(parts.sum()):, 0] == -1).all()
        work, seq = split_tables(np.full(B, 5000, dtype=np.int64), splits, 64)
        assert ((seq & 255) == min(splits, 32)).all()
    work, seq = split_tables(np.array([100, 100, 100, 30000], dtype=np.int64), 8, 64)
    assert (seq & 255).tolist()[3] >= 25


def test_generation_config_json_gives_defaults_and_more_stop_tokens(tmp_path):
    """do_sample / temperature / top_k / top_p and eos_token_id of generation_config.json, merged with the
    configuration's EOS ids (src/engine/generate.jl:83-93); greedy without the file or without do_sample."""
    import json
    from types import SimpleNamespace
    from tileinfer_b200.api import generation_defaults
    engine = SimpleNamespace(spec=SimpleNamespace(eos_token_ids=[2]))
    sampling, stop = generation_defaults(str(tmp_path), engine)
    assert sampling.greedy and stop == [2]
    (tmp_path / "generation_config.json").write_text(json.dumps(
        {"do_sample": True, "temperature": 0.6, "top_k": 20, "top_p": 0.95, "eos_token_id": [2, 7]}))
    sampling, stop = generation_defaults(str(tmp_path), engine)
    assert (sampling.temperature, sampling.top_k, sampling.top_p) == (0.6, 20, 0.95) and stop == [2, 7]
    (tmp_path / "generation_config.json").write_text(json.dumps({"temperature": 0.6, "eos_token_id": 9}))
    sampling, stop = generation_defaults(str(tmp_path), engine)
    assert sampling.greedy and stop == [2, 9]
    assert engine.spec.eos_token_ids == [2]                      # the configuration's own list is not changed
