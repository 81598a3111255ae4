"""The engine in-process: long decoding, first tokens, generation through the entry point, graph
replay against eager launches, stop tokens and slot reuse, errors that leave the cache untouched,
and the reference's own goldens."""
import os
import tempfile

import pytest
import torch

import helpers
import plain_apertus as plain

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def models():
    """Model folders for the tiny configurations, and the plain implementation's view of them."""
    import tileinfer_b200 as ti
    from tileinfer_b200.config import ApertusConfig
    from tileinfer_b200.weights import write_model_folder
    with tempfile.TemporaryDirectory() as d:
        out = {}
        for name, cfg_dict, seed in (("A", helpers.TINY_A, 0), ("B", helpers.TINY_B, 1), ("C", helpers.TINY_C, 2)):
            folder = write_model_folder(ApertusConfig.from_dict(cfg_dict), seed, os.path.join(d, name))
            out[name] = (folder,) + plain.load_folder(folder)
        out["fixture"] = (helpers.reference_fixture_folder(os.path.join(d, "fixture")),)
        yield out


def tolerance(dtype, ref):
    scale = max(float(ref.abs().max()), 1.0)
    return 2e-5 * scale if dtype == "float32" else 4 * float(ref.abs().max()) * 2.0 ** -8


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_long_decoding_and_first_tokens(models, name, dtype):
    """A prompt of ONE token, then 200 tokens one by one (crossing page borders at 64, 128, 192, and for B
    the rope-scaling threshold at 64), two sequences in the batch that start together."""
    import tileinfer_b200 as ti
    folder, pc, pw = models[name]
    eng = ti.load_model(folder, dtype=dtype, max_context=256, max_seqs=2)
    pdt = torch.float32 if dtype == "float32" else torch.bfloat16
    seqs = helpers.random_prompts(pc.vocab, [201, 150], 5)
    refs = [plain.forward(pc, pw, s, pdt) for s in seqs]
    slots = [eng.new_sequence(), eng.new_sequence()]
    worst = 0.0
    for pos in range(201):
        live = [i for i in range(2) if pos < len(seqs[i])]
        logits = eng.step([(slots[i], [seqs[i][pos]]) for i in live]).cpu()
        for row, i in enumerate(live):
            err = float((logits[row] - refs[i][pos]).abs().max())
            assert err <= tolerance(dtype, refs[i]), f"{name} {dtype} sequence {i} position {pos}: {err}"
            worst = max(worst, err)
    eng.check_health()
    assert eng.sequence_length(slots[0]) == 201 and eng.sequence_length(slots[1]) == 150


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_graph_replay_equals_eager_launches(models, dtype):
    """Decode steps replayed from CUDA graphs (kernels launched as programmatic dependents, overlapping
    their predecessors) give bit-identical logits to strictly serial eager launches, over 70 steps that
    cross a page border, with a batch that shrinks."""
    import tileinfer_b200 as ti
    from tileinfer_b200.kernels import library
    folder, pc, pw = models["B"]
    prompts = helpers.random_prompts(pc.vocab, [3, 60, 17], 7)
    feeds = helpers.random_prompts(pc.vocab, [70, 70, 70], 8)
    runs = []
    for graphs, pdl in ((True, True), (False, False)):
        library.set_pdl(pdl)
        try:
            eng = ti.Engine.load(folder, dtype=dtype, max_context=256, max_seqs=4, max_tokens=1024, graphs=graphs)
            slots = [eng.new_sequence() for _ in prompts]
            out = [eng.step(list(zip(slots, prompts))).clone()]
            for t in range(70):
                live = [i for i in range(3) if not (i == 1 and t >= 40)]       # sequence 1 leaves after 40 steps
                out.append(eng.step([(slots[i], [feeds[i][t]]) for i in live]).clone())
            runs.append(out)
            eng.check_health()
        finally:
            library.set_pdl(True)
    for a, b in zip(*runs):
        assert torch.equal(a, b)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_reference_goldens_through_the_engine(models, dtype):
    """The reference's own bars on its tiny checkpoint (test/model/forward.jl:138-146)."""
    import tileinfer_b200 as ti
    eng = ti.load_model(models["fixture"][0], dtype=dtype, max_context=128, max_seqs=1)
    for case in helpers.reference_goldens().values():
        ids, gold = case["ids"], case[dtype]
        s = eng.new_sequence()
        logits = eng.step([(s, ids)], [list(range(len(ids)))]).cpu()
        eng.free_sequence(s)
        for t in range(len(ids)):
            top, want = torch.tensor(gold["topk_ids"][t]), torch.tensor(gold["topk_logits"][t])
            err = float((logits[t][top] - want).abs().max())
            if dtype == "float32":
                assert err < 1e-4 and int(logits[t].argmax()) == gold["topk_ids"][t][0]
            else:
                assert err < 0.1
                if want[0] - want[1] >= 0.25:
                    assert int(logits[t].argmax()) == gold["topk_ids"][t][0]
        if dtype == "float32":
            assert ti.generate(eng, ids, max_new_tokens=24, stop_ids=[]) == gold["greedy"]


def test_greedy_generation_through_the_entry_point(models):
    """Batches of unequal prompts, more requests than slots (so batches follow one another and slots are
    used again), against the plain implementation's greedy continuation; 32-bit decides exactly."""
    import tileinfer_b200 as ti
    for name, lengths in (("A", [5, 9, 13]), ("B", [1, 4, 17, 33, 70])):
        folder, pc, pw = models[name]
        prompts = helpers.random_prompts(pc.vocab, lengths, 11)
        eng = ti.load_model(folder, dtype="float32", max_context=128, max_seqs=2)
        got = ti.generate(eng, prompts, max_new_tokens=8, stop_ids=[])
        assert got == [plain.generate(pc, pw, p, 8) for p in prompts]
        assert eng.cache.slots.held == 0 and eng.cache.free_pages() == eng.cache.num_pages
        assert ti.generate(eng, prompts[0], max_new_tokens=3, stop_ids=[]) == got[0][:3]      # one prompt in, one list out


def test_sampled_generation_and_stop_tokens(models):
    """Temperature / top-k / top-p sampling follows the plain rule token for token (32-bit logits, same
    seeds); a stop token ends its sequence early, is not returned, and frees the slot."""
    import tileinfer_b200 as ti
    from tileinfer_b200.sampling import SamplingParams, sequence_seed
    folder, pc, pw = models["B"]
    prompts = helpers.random_prompts(pc.vocab, [1, 4, 17, 33, 70], 12)
    eng = ti.load_model(folder, dtype="float32", max_context=128, max_seqs=8)
    for params in (SamplingParams(temperature=0.8), SamplingParams(temperature=1.0, top_k=20, top_p=0.9)):
        got = ti.generate(eng, prompts, max_new_tokens=12, sampling=params, stop_ids=[], seed=1234)
        want = [plain.generate(pc, pw, p, 12, temperature=params.temperature, top_k=params.top_k, top_p=params.top_p,
                               seed=sequence_seed(1234, i)) for i, p in enumerate(prompts)]
        assert got == want
    greedy = ti.generate(eng, prompts, max_new_tokens=12, stop_ids=[])
    stop = greedy[2][5]                                   # a token that request 2 emits as its sixth
    cut = ti.generate(eng, prompts, max_new_tokens=12, stop_ids=[stop])
    for g, c in zip(greedy, cut):
        assert c == (g[:g.index(stop)] if stop in g else g)
    assert len(cut[2]) <= 5
    assert eng.cache.slots.held == 0
    seen = []
    ti.generate(eng, prompts[:2], max_new_tokens=3, stop_ids=[], on_token=lambda r, t: seen.append((r, t)))
    assert len(seen) == 6 and {r for r, _ in seen} == {0, 1}


@pytest.mark.parametrize("params", [dict(temperature=0.0), dict(temperature=0.9, top_k=40, top_p=0.95)])
def test_the_one_call_decode_loop_gives_what_the_step_by_step_loop_gives(models, params):
    """With graphs the generation loop enqueues a step by ONE C++ call (sample, hand the ids over, reserve,
    upload, launch the graph); without graphs it does the same step by step from Python. 48 tokens for nine
    requests with stop tokens that several of them hit at different times (rows drop out, the sampler's
    seeds and counters are compacted on the device, pages are crossed): the same tokens, in 32-bit exactly."""
    import tileinfer_b200 as ti
    from tileinfer_b200.sampling import SamplingParams
    folder, pc, pw = models["B"]
    prompts = helpers.random_prompts(pc.vocab, [1, 4, 17, 33, 70, 9, 50, 2, 63], 31)
    sampling = SamplingParams(**params)
    outs = []
    for graphs in (True, False):
        eng = ti.Engine.load(folder, dtype="float32", max_context=128, max_seqs=9, max_tokens=9 * 128, graphs=graphs)
        free = ti.generate(eng, prompts, max_new_tokens=48, sampling=sampling, stop_ids=[], seed=77)
        if graphs:
            counts = {}
            for g in free:
                for t in set(g[3:]):
                    counts[t] = counts.get(t, 0) + 1
            stops = sorted(counts, key=lambda t: (-counts[t], t))[:4]
        cut = ti.generate(eng, prompts, max_new_tokens=48, sampling=sampling, stop_ids=stops, seed=77)
        again = ti.generate(eng, prompts, max_new_tokens=48, sampling=sampling, stop_ids=stops, seed=77)     # every graph captured by now
        assert again == cut and eng.cache.slots.held == 0 and eng.cache.free_pages() == eng.cache.num_pages
        outs.append((free, cut))
    assert outs[0] == outs[1]
    free, cut = outs[0]
    assert len({len(c) for c in cut}) > 2                                    # requests ended at different times
    for f, c in zip(free, cut):
        hit = [j for j, t in enumerate(f) if t in stops]
        assert c == (f[:hit[0]] if hit else f)


def test_errors_leave_the_cache_untouched(models):
    import tileinfer_b200 as ti
    from tileinfer_b200.cache import OutOfPagesError
    folder, pc, pw = models["A"]
    eng = ti.Engine.load(folder, dtype="float32", max_context=256, max_seqs=2, max_tokens=128)
    a, b = eng.new_sequence(), eng.new_sequence()
    eng.step([(a, [1] * 60)])
    free = eng.cache.free_pages()
    with pytest.raises(OutOfPagesError):
        eng.step([(a, [1] * 10), (b, [2] * 70)])          # needs 1 + 2 pages, 1 free
    assert eng.cache.free_pages() == free and eng.sequence_length(a) == 60 and eng.sequence_length(b) == 0
    with pytest.raises(ValueError, match="vocabulary"):
        eng.step([(a, [pc.vocab])])
    with pytest.raises(ValueError, match="twice"):
        eng.step([(a, [1]), (a, [2])])
    with pytest.raises(ValueError, match="max context"):
        eng.step([(b, [1] * 300)])
    ref = plain.forward(pc, pw, [1] * 60 + [3], torch.float32)[-1]
    assert float((eng.step([(a, [3])]).cpu()[0] - ref).abs().max()) < 2e-5     # still consistent afterwards


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rolling_a_sequence_back_and_feeding_the_tokens_again(models, dtype):
    """Engine.truncate drops a sequence's last positions; feeding the same tokens again gives the same logits
    bit for bit, also across a page's border (the page goes back to the pool and is taken again), as the
    reference does with truncate! + forward! (test/model/forward.jl:65-67)."""
    import tileinfer_b200 as ti
    folder, pc, pw = models["B"]
    eng = ti.Engine.load(folder, dtype=dtype, max_context=256, max_seqs=2, max_tokens=512)
    seq = helpers.random_prompts(pc.vocab, [70], 21)[0]
    ref = plain.forward(pc, pw, seq, torch.float32 if dtype == "float32" else torch.bfloat16)
    a, b = eng.new_sequence(), eng.new_sequence()
    eng.step([(b, seq[:30])])                                      # a neighbour that must not be disturbed
    eng.step([(a, seq[:60])])
    first = [eng.step([(a, [seq[t]]), (b, [seq[30 + t - 60]])]).clone() for t in range(60, 67)]
    free = eng.cache.free_pages()
    eng.truncate(a, 66)                                            # one token back
    assert eng.sequence_length(a) == 66 and eng.cache.free_pages() == free
    again = eng.step([(a, [seq[66]])])
    assert float((again[0].cpu() - ref[66]).abs().max()) <= tolerance(dtype, ref)
    if dtype == "float32":                                         # (in bfloat16 a step of one sequence splits its keys otherwise)
        assert torch.equal(again[0], first[6][0])
    eng.truncate(a, 62)                                            # back across the page border at 64
    assert eng.cache.free_pages() == free + 1
    redo = eng.step([(a, seq[62:67])], [[0, 1, 2, 3, 4]])          # five tokens in one step this time
    for j, t in enumerate(range(62, 67)):
        assert float((redo[j].cpu() - ref[t]).abs().max()) <= tolerance(dtype, ref)
        if dtype == "float32":
            assert torch.equal(redo[j], first[t - 60][0])
    assert float((eng.step([(b, [seq[37]])])[0].cpu() - ref[37]).abs().max()) <= tolerance(dtype, ref)
    with pytest.raises(ValueError, match="truncate"):
        eng.truncate(a, 68)
    eng.check_health()


def test_a_long_prompt_is_cut_into_chunks_without_changing_results(models):
    import tileinfer_b200 as ti
    folder, pc, pw = models["C"]
    prompts = helpers.random_prompts(pc.vocab, [150, 40, 99], 13)
    whole = ti.Engine.load(folder, dtype="float32", max_context=256, max_seqs=3, max_tokens=1024)
    cut = ti.Engine.load(folder, dtype="float32", max_context=256, max_seqs=3, max_tokens=1024, max_step_tokens=64)
    want = [[149, 3, 70], [39, 0], [50, 98]]             # in any order, also across the chunks' borders
    outs = []
    for eng in (whole, cut):
        slots = [eng.new_sequence() for _ in prompts]
        outs.append(eng.step(list(zip(slots, prompts)), want).cpu())
    assert torch.equal(outs[0], outs[1])
    ref = torch.stack([plain.forward(pc, pw, p, torch.float32)[w] for p, ws in zip(prompts, want) for w in ws])
    assert float((outs[0] - ref).abs().max()) < 2e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_in_chunks_through_the_tensor_core_attention(dtype):
    """1,500 tokens at head size 64 (the tensor-core prefill attention in bfloat16) in steps of at most
    512: the later chunks attend to over a thousand cached keys (many key steps, pages of earlier
    chunks), far beyond the 128 positions up to which this configuration's rotation is unscaled. Logits
    along the prompt and of a few decoded tokens against the plain implementation."""
    import tileinfer_b200 as ti
    from tileinfer_b200.config import ApertusConfig
    from tileinfer_b200.weights import write_model_folder
    with tempfile.TemporaryDirectory() as d:
        folder = write_model_folder(ApertusConfig.from_dict(dict(helpers.TINY_D, max_position_embeddings=2048)), 9, os.path.join(d, "m"))
        pc, pw = plain.load_folder(folder)
        prompt = helpers.random_prompts(pc.vocab, [1506], 15)[0]
        pdt = torch.float32 if dtype == "float32" else torch.bfloat16
        ref = plain.forward(pc, pw, prompt, pdt)
        eng = ti.Engine.load(folder, dtype=dtype, max_context=1536, max_seqs=1, max_tokens=1536, max_step_tokens=512)
        tol = tolerance(dtype, ref)
        a = eng.new_sequence()
        want = [0, 300, 511, 512, 1023, 1024, 1400, 1499]
        got = eng.step([(a, prompt[:1500])], [want]).cpu()
        assert float((got - ref[want]).abs().max()) <= tol
        for t in range(1500, 1506):
            row = eng.step([(a, [prompt[t]])]).cpu()[0]
            assert float((row - ref[t]).abs().max()) <= tol, t
        eng.check_health()


def test_a_group_wider_than_the_fast_attention_takes_falls_back_to_the_plain_kernel():
    """130 query heads on one KV head: more than the fast attention kernels take (128), so prompt and decode steps
    run the plain attention kernel, with the same logits as the plain implementation."""
    import tileinfer_b200 as ti
    from tileinfer_b200.config import ApertusConfig
    from tileinfer_b200.kernels import library
    from tileinfer_b200.weights import write_model_folder
    cfg = dict(helpers.TINY_A, num_attention_heads=130, num_key_value_heads=1, head_dim=16, hidden_size=72)
    with tempfile.TemporaryDirectory() as d:
        folder = write_model_folder(ApertusConfig.from_dict(cfg), 4, os.path.join(d, "m"))
        pc, pw = plain.load_folder(folder)
        prompts = helpers.random_prompts(pc.vocab, [70, 9], 5)
        refs = [plain.forward(pc, pw, p, torch.bfloat16) for p in prompts]
        eng = ti.Engine.load(folder, dtype="bfloat16", max_context=128, max_seqs=2)
        ids = [eng.new_sequence() for _ in prompts]
        before = dict(library.call_counts)
        got = eng.step([(i, p[:-3]) for i, p in zip(ids, prompts)], [[len(p) - 4] for p in prompts]).cpu()
        for n, (p, ref) in enumerate(zip(prompts, refs)):
            assert float((got[n] - ref[len(p) - 4]).abs().max()) <= tolerance("bfloat16", ref), n
        for t in range(3, 0, -1):
            rows = eng.step([(i, [p[-t]]) for i, p in zip(ids, prompts)]).cpu()
            for n, (p, ref) in enumerate(zip(prompts, refs)):
                assert float((rows[n] - ref[len(p) - t]).abs().max()) <= tolerance("bfloat16", ref), (n, t)
        used = {k for k, v in library.call_counts.items() if v > before.get(k, 0)}
        assert "ti_attention_plain" in used
        eng.check_health()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_more_sequences_in_a_decode_step_than_tokens_in_a_prompt_chunk(dtype):
    """40 sequences with prompt steps cut at 16 tokens: the prompts go through in several chunks, the one-token
    steps of all 40 together are never cut and have more tokens than any chunk. Logits of the prompts' last
    tokens and of four decode steps against the plain implementation."""
    import tileinfer_b200 as ti
    from tileinfer_b200.config import ApertusConfig
    from tileinfer_b200.weights import write_model_folder
    with tempfile.TemporaryDirectory() as d:
        folder = write_model_folder(ApertusConfig.from_dict(helpers.TINY_B), 21, os.path.join(d, "m"))
        pc, pw = plain.load_folder(folder)
        prompts = helpers.random_prompts(pc.vocab, [5 + (7 * i) % 11 for i in range(40)], 22)
        pdt = torch.float32 if dtype == "float32" else torch.bfloat16
        refs = [plain.forward(pc, pw, p, pdt) for p in prompts]
        eng = ti.Engine.load(folder, dtype=dtype, max_context=64, max_seqs=40, max_step_tokens=16)
        ids = [eng.new_sequence() for _ in prompts]
        got = eng.step([(i, p[:-4]) for i, p in zip(ids, prompts)], [[len(p) - 5] for p in prompts]).cpu()
        for n, (p, ref) in enumerate(zip(prompts, refs)):
            assert float((got[n] - ref[len(p) - 5]).abs().max()) <= tolerance(dtype, ref), n
        for t in range(4, 0, -1):
            rows = eng.step([(i, [p[-t]]) for i, p in zip(ids, prompts)]).cpu()
            for n, (p, ref) in enumerate(zip(prompts, refs)):
                assert float((rows[n] - ref[len(p) - t]).abs().max()) <= tolerance(dtype, ref), (n, t)
        eng.check_health()


@pytest.mark.parametrize("heads,kv_heads", [(20, 1), (36, 2)])
def test_many_query_heads_per_kv_head_run_the_fast_attention(heads, kv_heads):
    """20 and 18 query heads per KV head (more than the 16 a decode block takes at once): a prompt of 500
    tokens through the tensor-core prefill attention and two shorter ones beside it, then 12 decode steps
    of the three together, against the plain implementation; the fast kernels are the ones that ran."""
    import tileinfer_b200 as ti
    from tileinfer_b200.config import ApertusConfig
    from tileinfer_b200.kernels import library
    from tileinfer_b200.weights import write_model_folder
    cfg = dict(helpers.TINY_D, num_attention_heads=heads, num_key_value_heads=kv_heads, hidden_size=144, max_position_embeddings=2048)
    with tempfile.TemporaryDirectory() as d:
        folder = write_model_folder(ApertusConfig.from_dict(cfg), 12, os.path.join(d, "m"))
        pc, pw = plain.load_folder(folder)
        prompts = helpers.random_prompts(pc.vocab, [512, 45, 141], 16)
        refs = [plain.forward(pc, pw, p, torch.bfloat16) for p in prompts]
        eng = ti.Engine.load(folder, dtype="bfloat16", max_context=512, max_seqs=3)
        ids = [eng.new_sequence() for _ in prompts]
        before = dict(library.call_counts)
        got = eng.step([(i, p[:-12]) for i, p in zip(ids, prompts)], [[0, len(p) - 13] for p in prompts]).cpu()
        for n, (p, ref) in enumerate(zip(prompts, refs)):
            assert float((got[2 * n:2 * n + 2] - ref[[0, len(p) - 13]]).abs().max()) <= tolerance("bfloat16", ref), n
        for t in range(12, 0, -1):
            rows = eng.step([(i, [p[-t]]) for i, p in zip(ids, prompts)]).cpu()
            for n, (p, ref) in enumerate(zip(prompts, refs)):
                assert float((rows[n] - ref[len(p) - t]).abs().max()) <= tolerance("bfloat16", ref), (n, t)
        used = {k: v - before.get(k, 0) for k, v in library.call_counts.items() if v > before.get(k, 0)}
        assert used.get("ti_attention_prefill_tc") == pc.layers and used.get("ti_attention_decode_shared", 0) >= pc.layers
        assert "ti_attention_plain" not in used and "ti_attention_prefill" not in used
        eng.check_health()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_context_beyond_8192_positions_next_to_a_short_one(dtype):
    """9,000 positions (past the 8,192 of Apertus-8B's rope scaling record, 141 pages) next to a sequence of 300:
    the prompts go through in chunks of 2,048 tokens that attend to the earlier chunks' pages, then both
    sequences decode together, where the fast path shares the decode attention's work slots out by length (the
    long sequence is read by many blocks, the short one by one). In 32-bit a page that was skipped or read
    twice would move the logits by far more than the bound; bfloat16 checks the fast kernels on the same data."""
    import tileinfer_b200 as ti
    from tileinfer_b200.config import ApertusConfig
    from tileinfer_b200.weights import write_model_folder
    cfg_dict = dict(helpers.TINY_D, max_position_embeddings=16384, num_hidden_layers=1,
                    rope_scaling={"rope_type": "llama3", "factor": 8.0, "original_max_position_embeddings": 8192,
                                  "low_freq_factor": 1.0, "high_freq_factor": 4.0})
    with tempfile.TemporaryDirectory() as d:
        folder = write_model_folder(ApertusConfig.from_dict(cfg_dict), 17, os.path.join(d, "m"))
        pc, pw = plain.load_folder(folder)
        long_, short = helpers.random_prompts(pc.vocab, [9020, 320], 19)
        pdt = torch.float32 if dtype == "float32" else torch.bfloat16
        want_long = [0, 2047, 2048, 8191, 8192, 8999]
        ref_long, ref_short = plain.forward(pc, pw, long_, pdt), plain.forward(pc, pw, short, pdt)
        eng = ti.Engine.load(folder, dtype=dtype, max_context=9088, max_seqs=2, max_tokens=9088 + 384, max_step_tokens=2048)
        a, b = eng.new_sequence(), eng.new_sequence()
        got = eng.step([(a, long_[:9000]), (b, short[:300])], [want_long, [0, 299]]).cpu()
        tol_long, tol_short = tolerance(dtype, ref_long), tolerance(dtype, ref_short)
        assert float((got[:6] - ref_long[want_long]).abs().max()) <= tol_long
        assert float((got[6:] - ref_short[[0, 299]]).abs().max()) <= tol_short
        for t in range(20):
            row = eng.step([(a, [long_[9000 + t]]), (b, [short[300 + t]])]).cpu()
            assert float((row[0] - ref_long[9000 + t]).abs().max()) <= tol_long, t
            assert float((row[1] - ref_short[300 + t]).abs().max()) <= tol_short, t
        if dtype == "bfloat16":
            plan = eng.planner._layout(2, 2, 2)[1]["groups"][0].plan
            work, seq = plan.tables(2, eng.planner._layout(2, 2, 2)[1]["groups"][0].plan_table)
            parts = (seq.cpu() & 255).tolist()
            assert parts[0] > parts[1] >= 1                     # the long sequence got most of the work slots
        eng.check_health()


def test_command_line(models, capsys):
    from tileinfer_b200.cli import cli
    folder, pc, pw = models["A"]
    prompt = helpers.random_prompts(pc.vocab, [9], 14)[0]
    assert cli(["run", folder, " ".join(map(str, prompt)), "--max-tokens", "6", "--dtype", "float32", "--max-context", "64",
                "--stop-ids", ""]) == 0
    out = capsys.readouterr()
    assert [int(t) for t in out.out.split()] == plain.generate(pc, pw, prompt, 6)
    assert "9 prompt tokens, 6 generated" in out.err
    assert cli(["run", folder, "1 2", "--bogus", "1"]) == 1 and "unknown option --bogus" in capsys.readouterr().err
    assert cli(["run", folder]) == 1 and cli(["frobnicate"]) == 1 and cli([]) == 1 and cli(["help"]) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_layer_at_apertus_8b_sizes(dtype):
    """The layer sizes of Apertus-8B (hidden 4096, 32 / 8 heads of 128, intermediate 21504, llama3 RoPE
    with theta 12e6), one layer and a smaller vocabulary, against the plain implementation: a prompt
    whole, its last tokens one by one, and a batch of two unequal sequences. This is where the
    tensor-core product, the weight-streaming product and both attention kernels run at the sizes they
    were written for."""
    import tileinfer_b200 as ti
    from tileinfer_b200.config import ApertusConfig
    from tileinfer_b200.weights import write_model_folder
    cfg_dict = {
        "architectures": ["ApertusForCausalLM"], "model_type": "apertus", "num_hidden_layers": 1, "hidden_size": 4096,
        "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 21504, "vocab_size": 16384,
        "rope_theta": 12000000.0, "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "original_max_position_embeddings": 8192,
                                                  "low_freq_factor": 1.0, "high_freq_factor": 4.0},
        "rms_norm_eps": 1e-5, "qk_norm": True, "tie_word_embeddings": True, "hidden_act": "xielu", "max_position_embeddings": 4096,
    }
    with tempfile.TemporaryDirectory() as d:
        folder = write_model_folder(ApertusConfig.from_dict(cfg_dict), 5, os.path.join(d, "m"))
        pc, pw = plain.load_folder(folder)
        pdt = torch.float32 if dtype == "float32" else torch.bfloat16
        prompts = helpers.random_prompts(16384, [150, 37, 400], 6)
        refs = [plain.forward(pc, pw, p, pdt) for p in prompts]
        eng = ti.load_model(folder, dtype=dtype, max_context=512, max_seqs=2)
        tol = tolerance(dtype, refs[0])
        from tileinfer_b200.kernels import library
        before = dict(library.call_counts)
        a = eng.new_sequence()
        got = eng.step([(a, prompts[0][:142])], [list(range(142))]).cpu()
        assert float((got - refs[0][:142]).abs().max()) <= tol
        used = {k: v - before.get(k, 0) for k, v in library.call_counts.items() if v > before.get(k, 0)}
        if dtype == "bfloat16":                                        # the kernels written for these sizes did the work
            # 142 tokens: q|k|v, o and down on the 128-row product; the up projection and the head, whose k cannot be cut,
            # on the product with the tokens in the tensor-memory lanes (two halves of 128)
            assert used.get("ti_gemm_tcgen05") == 3 and used.get("ti_gemm_tcgen05_decode") == 2
            # a short prompt: the mma.sync attention (the tensor-memory kernel takes sequences beyond 384 positions, below)
            assert used.get("ti_attention_prefill") == 1 and "ti_attention_prefill_tc" not in used
            assert "ti_gemm_plain" not in used and "ti_attention_plain" not in used
        else:
            assert "ti_gemm_tcgen05" not in used and "ti_attention_prefill_tc" not in used
        for t in range(142, 150):                                      # the last tokens one by one
            row = eng.step([(a, [prompts[0][t]])]).cpu()[0]
            assert float((row - refs[0][t]).abs().max()) <= tol, t
        eng.free_sequence(a)
        a, b = eng.new_sequence(), eng.new_sequence()                  # a batch of two, in reused slots
        got = eng.step([(a, prompts[0]), (b, prompts[1])], [[0, 149], [36]]).cpu()
        want = torch.stack([refs[0][0], refs[0][149], refs[1][36]])
        assert float((got - want).abs().max()) <= tol
        eng.free_sequence(a)
        before = dict(library.call_counts)
        a = eng.new_sequence()                                         # 100 tokens: the product with the tokens in the tensor-memory lanes
        got = eng.step([(a, prompts[0][:100])], [list(range(100))]).cpu()
        assert float((got - refs[0][:100]).abs().max()) <= tol
        if dtype == "bfloat16":
            assert library.call_counts.get("ti_gemm_tcgen05_decode", 0) - before.get("ti_gemm_tcgen05_decode", 0) == 2   # up projection and head
        eng.free_sequence(a)
        eng.free_sequence(b)
        # 400 + 37 tokens in one step: the o and down products have fewer tiles of 256 x 256 than there are SM pairs and
        # come in k slices that the norms add up; a sequence of 400 positions takes the tensor-memory attention.
        a, b = eng.new_sequence(), eng.new_sequence()
        wanted = [0, 100, 255, 256, 399]
        before = dict(library.call_counts)
        got = eng.step([(a, prompts[2]), (b, prompts[1])], [wanted, [0, 36]]).cpu()
        want = torch.stack([refs[2][i] for i in wanted] + [refs[1][0], refs[1][36]])
        assert float((got - want).abs().max()) <= tolerance(dtype, refs[2])
        if dtype == "bfloat16":
            from tileinfer_b200.kernels import fast
            assert fast.tc_splits(4096, 21504, 437) > 1 and fast.tc_splits(4096, 4096, 437) > 1
            assert library.call_counts.get("ti_attention_prefill_tc", 0) - before.get("ti_attention_prefill_tc", 0) == 1
        eng.check_health()


def _odd(**kw):
    c = {k: v for k, v in helpers.TINY_A.items() if k != "eos_token_id"}
    c.update(kw)
    return c


ODD_SIZES = {
    "width 100 (a multiple of 4 only)": _odd(hidden_size=100, num_attention_heads=3, num_key_value_heads=1, head_dim=32,
                                           intermediate_size=172, vocab_size=333),
    "odd width, feed-forward and vocabulary": _odd(hidden_size=77, num_attention_heads=2, num_key_value_heads=2, head_dim=16,
                                                   intermediate_size=203, vocab_size=99),
    "head 80": _odd(hidden_size=160, num_attention_heads=4, num_key_value_heads=2, head_dim=80),
    "head 96, 3 per group": _odd(hidden_size=192, num_attention_heads=6, num_key_value_heads=2, head_dim=96),
    "head 112, 7 per group": _odd(hidden_size=128, num_attention_heads=7, num_key_value_heads=1, head_dim=112),
    "head 24 (no multiple of 16)": _odd(hidden_size=96, num_attention_heads=4, num_key_value_heads=2, head_dim=24),
    "head 256": _odd(hidden_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=256),
    "head 512": _odd(hidden_size=512, num_attention_heads=2, num_key_value_heads=1, head_dim=512),
    "32 per group": _odd(hidden_size=256, num_attention_heads=32, num_key_value_heads=1, head_dim=64),
    "40 heads in 8 groups of head 128": _odd(hidden_size=256, num_attention_heads=40, num_key_value_heads=8, head_dim=128),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", sorted(ODD_SIZES))
def test_every_size_is_taken_or_handed_to_a_kernel_that_takes_it(case, dtype):
    """Sizes outside what the tensor-core and vector kernels take (widths that are no multiple of 8, head
    sizes that are no multiple of 16 or above 256, groups that are no power of two) run through the
    general kernels instead: a prompt of two unequal sequences, then 8 tokens one by one."""
    import tileinfer_b200 as ti
    from tileinfer_b200.config import ApertusConfig
    from tileinfer_b200.weights import write_model_folder
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    with tempfile.TemporaryDirectory() as d:
        folder = write_model_folder(ApertusConfig.from_dict(ODD_SIZES[case]), 1, os.path.join(d, "m"))
        cfg, W = plain.load_folder(folder)
        prompts = helpers.random_prompts(cfg.vocab, [150, 37], 3)
        refs = [plain.forward(cfg, W, p, tdt) for p in prompts]
        eng = ti.load_model(folder, dtype=dtype, max_context=256, max_seqs=2)
        slots = [eng.new_sequence() for _ in prompts]
        head = [len(p) - 8 for p in prompts]
        out = eng.step([(s, p[:h]) for s, p, h in zip(slots, prompts, head)], [list(range(h)) for h in head]).cpu()
        row = 0
        for ref, h in zip(refs, head):
            assert float((out[row:row + h] - ref[:h]).abs().max()) <= tolerance(dtype, ref)
            row += h
        for t in range(8):
            out = eng.step([(s, [p[h + t]]) for s, p, h in zip(slots, prompts, head)]).cpu()
            for i, (ref, h) in enumerate(zip(refs, head)):
                assert float((out[i] - ref[h + t]).abs().max()) <= tolerance(dtype, ref), (t, i)
        eng.check_health()


def test_a_head_size_the_kernels_do_not_take_is_refused_when_the_model_is_built():
    """No kernel takes heads above 512 or of odd size: building the model says so, before any step runs."""
    import tileinfer_b200 as ti
    from tileinfer_b200.config import ApertusConfig
    for head_dim in (528, 1024):
        cfg = ApertusConfig.from_dict(_odd(hidden_size=64, num_attention_heads=2, num_key_value_heads=1, head_dim=head_dim))
        with pytest.raises(ValueError, match=f"head size {head_dim}"):
            ti.Engine.random(cfg, 0, dtype="float32", max_context=64, max_seqs=1, max_tokens=64)
