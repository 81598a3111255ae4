"""Random configurations run random schedules against the plain implementation: batches of unequal prompts with wanted
places in any order, prompts cut into chunks of a random size, one token at a time afterwards with requests ending at
different times, now and then a sequence rolled back by one token and fed again, one batch after another on the same
cache (so slots and pages are used again), with and without CUDA graphs. The seeds are fixed; each draws every size of
the configuration (heads, groups, head size, widths, vocabulary, layers, eps, rope scaling, tied head, q/k norm)."""
import os
import random
import tempfile

import numpy as np
import pytest
import torch

import plain_apertus as plain
from tileinfer_b200.config import ApertusConfig
from tileinfer_b200.weights import write_model_folder

pytestmark = pytest.mark.gpu


def random_config(rng):
    nkv = rng.choice([1, 2, 3, 4])
    cfg = {
        "architectures": ["ApertusForCausalLM"], "model_type": "apertus",
        "num_hidden_layers": rng.choice([1, 2, 3]), "hidden_size": rng.choice([64, 72, 96, 120, 136, 200, 256, 512]),
        "num_attention_heads": nkv * rng.choice([1, 2, 3, 4, 5, 8]), "num_key_value_heads": nkv,
        "head_dim": rng.choice([16, 32, 48, 64, 80, 96, 128]), "intermediate_size": rng.choice([104, 192, 200, 328, 520, 1536]),
        "vocab_size": rng.choice([97, 256, 301, 392, 1000, 2051]), "rope_theta": rng.choice([10000.0, 500000.0, 12000000.0]),
        "rms_norm_eps": rng.choice([1e-5, 1e-6, 3e-6]), "qk_norm": rng.random() < 0.7, "tie_word_embeddings": rng.random() < 0.4,
        "hidden_act": "xielu", "max_position_embeddings": 1024, "attention_bias": False, "mlp_bias": False,
    }
    if rng.random() < 0.6:
        cfg["rope_scaling"] = {"rope_type": "llama3", "factor": rng.choice([4.0, 8.0]),
                               "original_max_position_embeddings": rng.choice([32, 64, 128]),
                               "low_freq_factor": 1.0, "high_freq_factor": rng.choice([2.0, 4.0])}
    return cfg


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [3, 14, 25, 37, 112, 205, 333, 1012, 6, 28])      # the last two draw batches of up to 160 sequences
def test_a_random_schedule_matches_the_plain_implementation(seed, dtype_name):
    import tileinfer_b200 as ti
    rng = random.Random(seed)
    cfg_dict = random_config(rng)
    cfg = ApertusConfig.from_dict(cfg_dict)
    dtype = torch.float32 if dtype_name == "float32" else torch.bfloat16
    with tempfile.TemporaryDirectory() as d:
        folder = write_model_folder(cfg, seed, os.path.join(d, "m"))
        pc, pw = plain.load_folder(folder)
        max_seqs = rng.choice([2, 4, 8, 12, 20, 40, 160])
        max_step = rng.choice([32, 64, 100, 256, 8192])
        batches, most = [], 0
        for _ in range(rng.choice([2, 3])):
            reqs = []
            for _ in range(rng.randint(1, max_seqs)):
                total = rng.choice([1, 2, 3, 17, 63, 64, 65, 100, 127, 128, 129, 200, rng.randint(1, 260)])
                reqs.append(([rng.randrange(cfg.vocab_size) for _ in range(total)], min(total - 1, rng.choice([0, 1, 2, 5, 20, 40]))))
            batches.append(reqs)
            most = max(most, sum(-(-len(t) // 64) * 64 for t, _ in reqs))
        eng = ti.Engine.load(folder, dtype=dtype_name, max_tokens=most + 64 * rng.choice([0, 1, 3]), max_seqs=max_seqs, max_context=1024,
                             max_step_tokens=max_step, graphs=rng.random() < 0.8)
        what = f"seed {seed}, {cfg_dict}, steps of {max_step}"
        checked = 0
        for reqs in batches:
            refs = [plain.forward(pc, pw, t, dtype).numpy() for t, _ in reqs]
            scale = max(float(np.abs(r).max()) for r in refs)
            tol = 2e-5 * max(scale, 1.0) if dtype_name == "float32" else 4 * scale * 2.0 ** -8
            slots = [eng.new_sequence() for _ in reqs]
            entries, want, where = [], [], []
            for i, (s, (toks, dec)) in enumerate(zip(slots, reqs)):
                head = len(toks) - dec
                w = sorted(rng.sample(range(head), rng.randint(0, min(head, 4))))
                if rng.random() < 0.5 and head - 1 not in w:
                    w.append(head - 1)
                if rng.random() < 0.3:
                    rng.shuffle(w)
                entries.append((s, toks[:head]))
                want.append(w)
                where += [(i, p) for p in w]
            logits = eng.step(entries, want).cpu().numpy()
            assert logits.shape[0] == len(where)
            for row, (i, p) in zip(logits, where):
                assert float(np.abs(row - refs[i][p]).max()) <= tol, f"prompt position {p} of request {i}; {what}"
                checked += 1
            fed = {i: len(t) - dec for i, (t, dec) in enumerate(reqs)}
            live = [i for i, (t, dec) in enumerate(reqs) if dec > 0]
            for i, (t, dec) in enumerate(reqs):
                if dec == 0:
                    eng.free_sequence(slots[i])
            while live:
                if rng.random() < 0.1:                        # roll one sequence back by a token: it is fed again below
                    i = rng.choice(live)
                    if fed[i] >= 2:
                        eng.truncate(slots[i], fed[i] - 1)
                        fed[i] -= 1
                out = eng.step([(slots[i], [reqs[i][0][fed[i]]]) for i in live]).cpu().numpy()
                for row, i in zip(out, live):
                    assert float(np.abs(row - refs[i][fed[i]]).max()) <= tol, f"position {fed[i]} of request {i} in a step of {len(live)}; {what}"
                    checked += 1
                    fed[i] += 1
                for i in [i for i in live if fed[i] >= len(reqs[i][0])]:
                    eng.free_sequence(slots[i])
                live = [i for i in live if fed[i] < len(reqs[i][0])]
            eng.check_health()
        assert checked > 0 and eng.cache.slots.held == 0 and eng.cache.free_pages() == eng.cache.num_pages


def kernel_size_config(rng):
    """Sizes that the tensor-core kernels take: heads of 64 or 128, 1 to 16 query heads per KV head (3, 5, 6, 7 and 12 among them,
    which do not divide a tile's 128 rows), widths of 1,024 to 3,072."""
    nkv = rng.choice([1, 2, 4, 8])
    return {"architectures": ["ApertusForCausalLM"], "model_type": "apertus", "num_hidden_layers": rng.choice([1, 2]),
            "hidden_size": rng.choice([1024, 1536, 2048, 3072]), "num_attention_heads": nkv * rng.choice([1, 2, 3, 4, 5, 6, 7, 8, 12, 16]),
            "num_key_value_heads": nkv, "head_dim": rng.choice([64, 128]), "intermediate_size": rng.choice([2048, 4096, 5120, 8192]),
            "vocab_size": rng.choice([1000, 4099, 32000]), "rope_theta": 500000.0, "rms_norm_eps": 1e-5, "qk_norm": rng.random() < 0.8,
            "tie_word_embeddings": rng.random() < 0.5, "hidden_act": "xielu", "max_position_embeddings": 2048,
            "attention_bias": False, "mlp_bias": False}


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [41, 44, 46, 53, 68])      # groups of 3, 7, 16, 12, 7; one to five prompts; steps of 200 to 2,843 tokens
def test_prompts_of_some_hundred_tokens_at_the_kernels_sizes(seed, dtype_name):
    """One to five prompts of 130 to 900 tokens in one step (cut into steps of 512 tokens for some seeds), then a few tokens
    one by one, at sizes where the step runs on the tensor-core products (k slices on SM pairs, the product with the
    tokens in the tensor-memory lanes up to 256 tokens) and on both prefill attention kernels, against the plain
    implementation."""
    import tileinfer_b200 as ti
    rng = random.Random(seed)
    cfg_dict = kernel_size_config(rng)
    cfg = ApertusConfig.from_dict(cfg_dict)
    dtype = torch.float32 if dtype_name == "float32" else torch.bfloat16
    with tempfile.TemporaryDirectory() as d:
        folder = write_model_folder(cfg, seed, os.path.join(d, "m"))
        pc, pw = plain.load_folder(folder)
        reqs = []
        for _ in range(rng.choice([1, 1, 2, 3, 5])):
            total = rng.choice([130, 200, 257, 300, 385, 449, 512, 640, 777, 900])
            reqs.append(([rng.randrange(cfg.vocab_size) for _ in range(total)], rng.choice([0, 1, 3])))
        eng = ti.Engine.load(folder, dtype=dtype_name, max_tokens=sum(-(-len(t) // 64) * 64 for t, _ in reqs) + 64, max_seqs=len(reqs),
                             max_context=1024, max_step_tokens=rng.choice([512, 8192]))
        refs = [plain.forward(pc, pw, t, dtype).numpy() for t, _ in reqs]
        scale = max(float(np.abs(r).max()) for r in refs)
        tol = 2e-5 * max(scale, 1.0) if dtype_name == "float32" else 4 * scale * 2.0 ** -8
        slots = [eng.new_sequence() for _ in reqs]
        want = [sorted(rng.sample(range(len(t) - dec), 3)) + [len(t) - dec - 1] for t, dec in reqs]
        logits = eng.step([(s, t[:len(t) - dec]) for s, (t, dec) in zip(slots, reqs)], want).cpu().numpy()
        row = 0
        for i, w in enumerate(want):
            for p in w:
                assert float(np.abs(logits[row] - refs[i][p]).max()) <= tol, f"request {i} position {p}; seed {seed}, {cfg_dict}"
                row += 1
        fed = [len(t) - dec for t, dec in reqs]
        live = [i for i, (t, dec) in enumerate(reqs) if dec]
        while live:
            out = eng.step([(slots[i], [reqs[i][0][fed[i]]]) for i in live]).cpu().numpy()
            for r, i in zip(out, live):
                assert float(np.abs(r - refs[i][fed[i]]).max()) <= tol, f"request {i} position {fed[i]}; seed {seed}, {cfg_dict}"
                fed[i] += 1
            live = [i for i in live if fed[i] < len(reqs[i][0])]
        eng.check_health()
