"""Decode steps of 9 to 100 sequences through the engine, with CUDA graphs on.

A batch of 100 unequal requests is prefilled together and then decoded one token each for 72 steps
while requests end at different times, so that the batch passes through the sizes
100 -> 65 -> 64 -> 33 -> 32 -> 9 -> 8 -> 1: every boundary at which the library changes kernel (the
weight-streaming product up to 8 tokens, the tensor-core product with token tiles of 32 and 64 and k
slices, the product with the tokens in the tensor-memory lanes from 65, decode attention with and
without splits). A second batch of 64 follows on the same cache, in the slots and pages the first
gave back. Every logit is compared with the plain implementation; in 32-bit every logit also equals,
bit for bit, the one the same request gives when it runs alone and whole.

AntoineBut/TileInfer.jl checks its one-sequence loop the same way: prefill, then steps of one token
against the one-shot run (test/model/forward.jl:43-68), and the pipelined loop against the plain one
(test/engine/runner.jl:44-93).
"""
import os
import random
import tempfile

import pytest
import torch

import helpers
import plain_apertus as plain

pytestmark = pytest.mark.gpu

LAYER_8B = {
    "architectures": ["ApertusForCausalLM"], "model_type": "apertus", "num_hidden_layers": 1, "hidden_size": 4096,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 21504, "vocab_size": 16384,
    "rope_theta": 12000000.0, "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "original_max_position_embeddings": 8192,
                                              "low_freq_factor": 1.0, "high_freq_factor": 4.0},
    "rms_norm_eps": 1e-5, "qk_norm": True, "tie_word_embeddings": True, "hidden_act": "xielu", "max_position_embeddings": 4096,
}
# (requests, tokens each decodes): the live count per step is the number of requests that decode at least that many.
FIRST = [(35, 3), (1, 5), (31, 8), (1, 10), (23, 13), (1, 15), (7, 40), (1, 72)]          # 100, 65, 64, 33, 32, 9, 8, 1
SECOND = [(44, 2), (4, 4), (7, 6), (6, 9), (2, 12), (1, 20)]                             # 64, 20, 16, 9, 3, 1


def make_requests(plan, vocab, seed):
    """Full token lists and how many of their last tokens are decoded one by one; prompts of 1 to 70 tokens,
    the lengths at a page's border among them."""
    rng = random.Random(seed)
    decode = [d for count, d in plan for _ in range(count)]
    rng.shuffle(decode)
    fixed = [1, 63, 64, 65, 2, 70]
    requests = []
    for i, d in enumerate(decode):
        prompt = fixed[i] if i < len(fixed) else rng.randint(1, 70)
        requests.append(([rng.randrange(vocab) for _ in range(prompt + d)], d))
    return requests


def tolerance(dtype, ref):
    scale = float(ref.abs().max())
    return 2e-5 * max(scale, 1.0) if dtype == "float32" else 4 * scale * 2.0 ** -8


def run_batch(eng, requests, refs, dtype, sizes_seen):
    """Prefill together, decode to the end; returns {(request, position): logits row} (device tensors)."""
    slots = [eng.new_sequence() for _ in requests]
    fed = [len(t) - d for t, d in requests]
    rows = {}
    logits = eng.step([(slots[i], t[:fed[i]]) for i, (t, _) in enumerate(requests)]).clone()
    for i in range(len(requests)):
        rows[(i, fed[i] - 1)] = logits[i]
    live = [i for i, (t, _) in enumerate(requests) if fed[i] < len(t)]
    for i in range(len(requests)):
        if i not in live:
            eng.free_sequence(slots[i])
    while live:
        sizes_seen.add(len(live))
        logits = eng.step([(slots[i], [requests[i][0][fed[i]]]) for i in live]).clone()
        for row, i in enumerate(live):
            rows[(i, fed[i])] = logits[row]
            fed[i] += 1
        for i in live:
            if fed[i] == len(requests[i][0]):
                eng.free_sequence(slots[i])                       # a request that ends gives its slot and pages back at once
        live = [i for i in live if fed[i] < len(requests[i][0])]
    eng.check_health()
    for (i, pos), row in rows.items():
        ref = refs[i]
        err = float((row.cpu() - ref[pos]).abs().max())
        assert err <= tolerance(dtype, ref), f"{dtype} request {i} position {pos} of {len(ref)}: |d| = {err}"
    return rows


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("model", ["tiny D", "one layer of Apertus-8B sizes"])
def test_large_decode_batches_that_shrink_through_every_kernel_boundary(model, dtype):
    import tileinfer_b200 as ti
    from tileinfer_b200.config import ApertusConfig
    from tileinfer_b200.kernels import library
    from tileinfer_b200.weights import write_model_folder
    cfg_dict = helpers.TINY_D if model == "tiny D" else LAYER_8B
    pdt = torch.float32 if dtype == "float32" else torch.bfloat16
    with tempfile.TemporaryDirectory() as d:
        folder = write_model_folder(ApertusConfig.from_dict(cfg_dict), 21, os.path.join(d, "m"))
        pc, pw = plain.load_folder(folder)
        eng = ti.Engine.load(folder, dtype=dtype, max_context=256, max_seqs=100, max_tokens=100 * 192, graphs=True)
        before = dict(library.call_counts)
        sizes = set()
        for plan, seed in ((FIRST, 31), (SECOND, 32)):
            requests = make_requests(plan, pc.vocab, seed)
            refs = [plain.forward(pc, pw, t, pdt) for t, _ in requests]
            rows = run_batch(eng, requests, refs, dtype, sizes)
            assert eng.cache.slots.held == 0 and eng.cache.free_pages() == eng.cache.num_pages
            if dtype == "float32":
                # Alone and whole, in a slot the batch used: the same bits as inside the batch.
                for i in sorted({i for i, _ in rows})[::7]:
                    s = eng.new_sequence()
                    t = requests[i][0]
                    whole = eng.step([(s, t)], [list(range(len(t)))])
                    eng.free_sequence(s)
                    for (j, pos), row in rows.items():
                        if j == i:
                            assert torch.equal(row, whole[pos]), f"request {i} position {pos} differs from its whole run"
        assert {100, 65, 64, 33, 32, 20, 16, 9, 8, 3, 1} <= sizes
        used = {k: v - before.get(k, 0) for k, v in library.call_counts.items() if v > before.get(k, 0)}
        plan = eng.planner._layout(1, 1, 1)[1]["groups"][0].plan           # the attention mixer's (bfloat16 only)
        splits = {B: plan.splits(B) if plan is not None else 1 for B in sizes}
        if dtype == "bfloat16" and model != "tiny D":
            # The kernels written for these sizes did the work: none of the plain ones ran.
            for name in ("ti_gemv_bf16", "ti_gemm_tcgen05", "ti_gemm_tcgen05_decode", "ti_attention_decode_shared"):
                assert used.get(name, 0) > 0, (name, used)
            assert used.get("ti_attention_prefill", 0) + used.get("ti_attention_prefill_tc", 0) > 0      # short prompts: the mma.sync kernel
            assert "ti_gemm_plain" not in used and "ti_attention_plain" not in used
            # Decode attention without splits (19 sequences and more at 8 KV heads) and with them.
            assert all(splits[B] == 1 for B in (100, 65, 64, 33, 32, 20)) and all(splits[B] > 1 for B in (9, 8, 3, 1))
        if dtype == "float32":
            assert not any(k in used for k in ("ti_gemv_bf16", "ti_gemm_tcgen05", "ti_gemm_tcgen05_decode"))


def test_graphs_of_other_batch_sizes_survive_a_reallocated_work_space():
    """Decoding at batch 8, then 7 (whose decode attention has MORE split rows than batch 8's: its work
    space grows and the old one is freed), then 8 again: the batch-8 graph captured before must not be
    replayed, since it writes into the freed buffer. Tensors allocated in between (which the allocator
    places in that freed memory) must keep their contents, and logits must equal eager launches."""
    import tileinfer_b200 as ti
    from tileinfer_b200.config import ApertusConfig
    from tileinfer_b200.weights import write_model_folder
    cfg_dict = dict(helpers.TINY_A, num_attention_heads=8, num_key_value_heads=8, head_dim=16, hidden_size=128,
                    max_position_embeddings=1024)
    with tempfile.TemporaryDirectory() as d:
        folder = write_model_folder(ApertusConfig.from_dict(cfg_dict), 4, os.path.join(d, "m"))
        prompts = helpers.random_prompts(cfg_dict["vocab_size"], [5, 9, 2, 30, 7, 11, 3, 4, 6], 3)
        feeds = helpers.random_prompts(cfg_dict["vocab_size"], [12] * 9, 4)
        outs = []
        for graphs in (True, False):
            eng = ti.Engine.load(folder, dtype="bfloat16", max_context=1024, max_seqs=9, max_tokens=9 * 1024, graphs=graphs)
            slots = [eng.new_sequence() for _ in prompts]
            got = [eng.step(list(zip(slots[:8], prompts[:8]))).clone()]
            guards = []
            for t in range(12):
                if t < 3:
                    live = list(range(8))                      # batch 8: captured at t = 0
                elif t < 6:
                    live = list(range(7))                      # batch 7: its first step enlarges the split work space
                else:
                    live = list(range(7)) + [8]                # batch 8 again
                if t == 6:
                    eng.step([(slots[8], prompts[8])])
                    if graphs:
                        work = eng.rt._buffers["attention.ws_o"]
                        assert work.numel() >= 7 * 5 * 8 * 16           # grew for batch 7 (5 splits) beyond batch 8's 4
                    # Fill the allocator's free blocks of the old work spaces' sizes, and fragments of them, with a pattern.
                    for count, copies in ((8 * 4 * 8 * 16, 64), (8 * 4 * 8 * 2, 64), (128, 256)):
                        guards += [torch.full((count,), 12345.0, dtype=torch.float32, device="cuda") for _ in range(copies)]
                got.append(eng.step([(slots[i], [feeds[i][t]]) for i in live]).clone())
            torch.cuda.synchronize()
            assert all(bool((g == 12345.0).all()) for g in guards), "a replayed graph wrote into memory it no longer owns"
            eng.check_health()
            outs.append(got)
        for a, b in zip(*outs):
            assert torch.equal(a, b)


def test_stop_tokens_in_bfloat16_with_the_next_step_in_flight():
    """Generation in bfloat16 on the fast kernels with stop tokens: a request that samples a stop token
    has already been put on the stream for one more step; its slot is freed while that step runs. The
    stop token is never returned, every returned token is the plain implementation's best token (or
    within rounding of it), a request that ended early ended on the stop token, and no slot is lost."""
    import tileinfer_b200 as ti
    from tileinfer_b200.config import ApertusConfig
    from tileinfer_b200.weights import write_model_folder
    with tempfile.TemporaryDirectory() as d:
        folder = write_model_folder(ApertusConfig.from_dict(helpers.TINY_B), 1, os.path.join(d, "m"))
        pc, pw = plain.load_folder(folder)
        prompts = helpers.random_prompts(pc.vocab, [1, 4, 17, 33, 70, 9, 12, 3, 8, 21, 2, 40], 12)
        eng = ti.load_model(folder, dtype="bfloat16", max_context=128, max_seqs=12)
        greedy = ti.generate(eng, prompts, max_new_tokens=16, stop_ids=[])
        counts = {}
        for g in greedy:
            for t in set(g[2:]):
                counts[t] = counts.get(t, 0) + 1
        stops = sorted(counts, key=lambda t: (-counts[t], t))[:3]             # tokens that several requests emit
        cut = ti.generate(eng, prompts, max_new_tokens=16, stop_ids=stops)
        assert eng.cache.slots.held == 0 and eng.cache.free_pages() == eng.cache.num_pages
        assert any(len(c) < 16 for c in cut)
        for p, c in zip(prompts, cut):
            assert not set(c) & set(stops)
            ref = plain.forward(pc, pw, p + c, torch.bfloat16)
            tol = 2 * 4 * float(ref.abs().max()) * 2.0 ** -8                  # the engine's and the plain logits both round
            for j in range(len(c) + (1 if len(c) < 16 else 0)):
                row = ref[len(p) - 1 + j]
                if j < len(c):
                    assert float(row.max() - row[c[j]]) <= tol, (j, c[j])
                else:                                                         # ended early: on a stop token
                    assert float(row.max() - row[stops].max()) <= tol
