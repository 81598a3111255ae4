"""The plain implementation against the reference's committed goldens (Hugging Face transformers'
ApertusForCausalLM on the reference's tiny checkpoint), with the reference's own bars
(test/model/forward.jl:138-146)."""
import tempfile

import pytest
import torch

import helpers
import plain_apertus as plain


@pytest.fixture(scope="module")
def fixture_model():
    with tempfile.TemporaryDirectory() as d:
        yield plain.load_folder(helpers.reference_fixture_folder(d))


@pytest.mark.parametrize("case", ["short", "medium", "long"])
def test_float32_matches_reference_goldens(fixture_model, case):
    cfg, W = fixture_model
    c = helpers.reference_goldens()[case]
    ids, gold = c["ids"], c["float32"]
    logits = plain.forward(cfg, W, ids, torch.float32)
    for t in range(len(ids)):
        top = torch.tensor(gold["topk_ids"][t])
        assert (logits[t][top] - torch.tensor(gold["topk_logits"][t])).abs().max() < 1e-4
        assert int(logits[t].argmax()) == gold["topk_ids"][t][0]
    if case != "long":
        assert plain.generate(cfg, W, ids, 24, torch.float32) == gold["greedy"]


@pytest.mark.parametrize("case", ["short", "medium"])
def test_bfloat16_matches_reference_goldens(fixture_model, case):
    cfg, W = fixture_model
    c = helpers.reference_goldens()[case]
    ids, gold = c["ids"], c["bfloat16"]
    logits = plain.forward(cfg, W, ids, torch.bfloat16)
    for t in range(len(ids)):
        top = torch.tensor(gold["topk_ids"][t])
        want = torch.tensor(gold["topk_logits"][t])
        assert (logits[t][top] - want).abs().max() < 0.1
        if want[0] - want[1] >= 0.25:
            assert int(logits[t].argmax()) == gold["topk_ids"][t][0]
