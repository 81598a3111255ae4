"""Trace replay through bin/trace_run: the same requests whole, with the last 32 tokens one by one,
and in batches of unequal lengths one after another (so that slots and pages are used again), in
32-bit and in bfloat16, against the plain implementation."""
import os
import tempfile

import numpy as np
import pytest
import torch

import helpers
import plain_apertus as plain
from replay_util import Trace, run_trace
from tileinfer_b200.config import ApertusConfig
from tileinfer_b200.weights import write_model_folder

pytestmark = pytest.mark.gpu

# Two layers with the layer sizes of Apertus-8B and its vocabulary, untied: the sizes the tensor-core products, the
# weight-streaming product and both attention kernels were written for.
LAYERS_8B = {
    "architectures": ["ApertusForCausalLM"], "model_type": "apertus", "num_hidden_layers": 2, "hidden_size": 4096,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 21504, "vocab_size": 131072,
    "rope_theta": 12000000.0, "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "original_max_position_embeddings": 8192,
                                              "low_freq_factor": 1.0, "high_freq_factor": 4.0},
    "rms_norm_eps": 1e-5, "qk_norm": True, "tie_word_embeddings": False, "hidden_act": "xielu", "max_position_embeddings": 4096,
}
CASES = {
    "8B layers": (LAYERS_8B, 4, [3, 70, 130, 33]),
    "A": (helpers.TINY_A, 0, [5, 9, 13, 40, 70, 33, 100]),
    "B": (helpers.TINY_B, 1, [1, 4, 17, 33, 70, 129, 64]),
    "D": (helpers.TINY_D, 3, [3, 70, 130, 200, 64, 450, 31]),       # head size 64: the tensor-core prefill attention (beyond 384 positions)
}


@pytest.fixture(scope="module", params=sorted(CASES))
def case(request):
    cfg_dict, seed, lengths = CASES[request.param]
    cfg = ApertusConfig.from_dict(cfg_dict)
    with tempfile.TemporaryDirectory() as d:
        folder = write_model_folder(cfg, seed, os.path.join(d, "model"))
        pc, pw = plain.load_folder(folder)
        prompts = helpers.random_prompts(cfg.vocab_size, lengths, seed + 10)
        requests = {f"r{i}": p for i, p in enumerate(prompts)}
        refs = {}
        for dtype in (torch.float32, torch.bfloat16):
            refs[dtype] = {r: plain.forward(pc, pw, t, dtype).numpy() for r, t in requests.items()}
        yield cfg, folder, requests, refs, d


def build_trace(requests):
    t = Trace()
    t.whole(requests)
    t.tail_one_by_one(requests)
    names = list(requests)
    # Two batches after one another; the second reuses the slots and pages of the first.
    b1, b2 = names[:4], names[3:] if len(names) > 4 else names[1:]
    dec = lambda group: {r: min(len(requests[r]) - 1, 3 + 5 * i) for i, r in enumerate(group)}
    t.batch({r: requests[r] for r in b1}, dec(b1), tag="x")
    t.batch({r: requests[r] for r in b2}, dec(b2), tag="y")
    t.batch({r: requests[r] for r in reversed(names)}, {r: min(len(requests[r]) - 1, 32) for r in names}, tag="z")
    return t


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_way_of_cutting_matches_the_plain_implementation(case, dtype):
    cfg, folder, requests, refs, tmp = case
    trace = build_trace(requests)
    # Most tokens held at once: the last batch holds every request, each rounded up to 64.
    max_tokens = sum(-(-len(t) // 64) * 64 for t in requests.values())
    got = run_trace(folder, dtype, trace, os.path.join(tmp, "out_" + dtype), max_tokens, cfg.vocab_size)
    ref = refs[torch.float32 if dtype == "float32" else torch.bfloat16]
    scale = max(float(np.abs(r).max()) for r in ref.values())
    tol = 2e-5 * max(scale, 1.0) if dtype == "float32" else 4 * scale * 2.0 ** -8
    worst = {}
    for (rid, pos), row in got.items():
        tag, r = rid[0], rid[1:]
        err = float(np.abs(row - ref[r][pos]).max())
        assert err <= tol, f"{dtype} request {rid} position {pos}: |d| = {err} > {tol}"
        worst[tag] = max(worst.get(tag, 0.0), err)
    assert set(worst) == {"w", "t", "x", "y", "z"}
    # Every position of every request was produced by every way of cutting.
    for tag in "wtz":
        assert sum(1 for (rid, _) in got if rid[0] == tag) == sum(len(t) for t in requests.values())
    if dtype == "float32":
        # The 32-bit kernels sum in an order that depends on the position alone: all cuts agree exactly.
        for (rid, pos), row in got.items():
            if rid[0] != "w":
                assert np.array_equal(row, got[("w" + rid[1:], pos)]), f"{rid} position {pos} differs from the whole run"
