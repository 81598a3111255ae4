"""A cache group with a window, end to end: an architecture defined in this file (Apertus layers, one of
them seeing only its last keys) runs through the engine against the plain implementation while the pages
that fell out of the window are given back, used again and, while free, filled with huge values."""
import dataclasses
import os
import tempfile

import pytest
import torch

import helpers
import plain_apertus as plain

pytestmark = pytest.mark.gpu

WINDOWS = (0, 100, 37)            # per layer; neither a multiple of the page size (64) nor of 16


def windowed_architecture():
    from tileinfer_b200.config import ApertusConfig, register_architecture

    @dataclasses.dataclass(frozen=True)
    class WindowedConfig:
        base: ApertusConfig
        windows: tuple

        @classmethod
        def from_dict(cls, c):
            return cls(ApertusConfig.from_dict(c), tuple(c["layer_windows"]))

        def to_dict(self):
            return {**self.base.to_dict(), "architectures": ["WindowedToyForCausalLM"], "layer_windows": list(self.windows)}

        def model_spec(self):
            spec = self.base.model_spec()
            layers = tuple(dataclasses.replace(l, mixer=dataclasses.replace(l.mixer, window=w or None))
                           for l, w in zip(spec.layers, self.windows))
            return dataclasses.replace(spec, architecture="WindowedToyForCausalLM", layers=layers)

    register_architecture("WindowedToyForCausalLM", WindowedConfig)
    return WindowedConfig


def poison_free_pages(engine, value=float("nan")):
    """Whatever no sequence holds is overwritten: a kernel that still reads a page which was given back
    (or one that was never taken) shows at once, and so does a page whose last user's values reach the
    next one."""
    for g in engine.cache.paged_groups:
        free = torch.tensor([p for p in range(g.num_pages) if not g.pages.is_held(p)], dtype=torch.long, device=g.k.device)
        if len(free):
            g.k[:, free] = value
            g.v[:, free] = -value


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_windowed_layers_release_pages_and_match_the_plain_implementation(dtype):
    from tileinfer_b200.engine import Engine
    from tileinfer_b200.weights import write_model_folder
    WindowedConfig = windowed_architecture()
    base = dict(helpers.TINY_D, num_hidden_layers=3, max_position_embeddings=2048)
    cfg = WindowedConfig.from_dict({**base, "layer_windows": list(WINDOWS)})
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    with tempfile.TemporaryDirectory() as d:
        folder = write_model_folder(cfg, 11, os.path.join(d, "w"))
        pcfg, W = plain.load_folder(folder)
        prompts = helpers.random_prompts(pcfg.vocab, [700, 333, 64], 5)
        refs = [plain.forward(pcfg, W, p, tdt, windows=WINDOWS) for p in prompts]

        def limit(ref):
            return 2e-5 * max(float(ref.abs().max()), 1.0) if dtype == "float32" else helpers.bf16_logit_tolerance(ref)

        # Steps of at most 128 tokens: the windowed groups hold a long prompt chunk by chunk.
        eng = Engine.load(folder, dtype=dtype, max_context=1024, max_seqs=3, max_tokens=3 * 1024, max_step_tokens=128,
                          graphs=False)
        full = [g for g in eng.cache.paged_groups if not g.window]
        win = sorted((g for g in eng.cache.paged_groups if g.window), key=lambda g: g.window)
        assert [g.window for g in win] == [37, 100] and len(full) == 1
        assert win[0].num_pages < win[1].num_pages < full[0].num_pages == 48
        for round_ in range(2):                                  # the second round runs in pages that were used before
            slots = [eng.new_sequence() for _ in prompts]
            poison_free_pages(eng)
            head = [len(p) - 32 for p in prompts]
            out = eng.step([(s, p[:h]) for s, p, h in zip(slots, prompts, head)], [list(range(h)) for h in head]).cpu()
            row = 0
            for ref, h in zip(refs, head):
                assert float((out[row:row + h] - ref[:h]).abs().max()) <= limit(ref)
                row += h
            for g in win:                                        # what is held: the window's pages and the release unit's slack
                assert g.pages.held <= sum(-(-(g.window - 1) // 64) + 3 for _ in prompts)
            assert full[0].pages.held == sum(-(-h // 64) for h in head)
            for t in range(32):
                poison_free_pages(eng)
                out = eng.step([(s, [p[h + t]]) for s, p, h in zip(slots, prompts, head)]).cpu()
                for i, (ref, h) in enumerate(zip(refs, head)):
                    assert float((out[i] - ref[h + t]).abs().max()) <= limit(ref), (round_, t, i)
            for s in slots:
                eng.free_sequence(s)
            assert all(g.pages.held == 0 for g in eng.cache.paged_groups)

        # Whole prompts in one step on an engine of its own: nothing is released before it was read.
        big = Engine.load(folder, dtype=dtype, max_context=1024, max_seqs=3, max_tokens=3 * 1024, graphs=False)
        slots = [big.new_sequence() for _ in prompts]
        poison_free_pages(big)
        out = big.step(list(zip(slots, prompts)), [list(range(len(p))) for p in prompts]).cpu()
        row = 0
        for ref, p in zip(refs, prompts):
            assert float((out[row:row + len(p)] - ref).abs().max()) <= limit(ref)
            row += len(p)


def test_decoding_with_graphs_far_beyond_a_window():
    """200 tokens one by one from CUDA graphs through layers whose windows they leave several times over;
    the windowed groups never hold more than their windows' pages."""
    from tileinfer_b200.engine import Engine
    from tileinfer_b200.weights import write_model_folder
    WindowedConfig = windowed_architecture()
    cfg = WindowedConfig.from_dict({**dict(helpers.TINY_D, num_hidden_layers=3), "layer_windows": list(WINDOWS)})
    with tempfile.TemporaryDirectory() as d:
        folder = write_model_folder(cfg, 12, os.path.join(d, "w"))
        pcfg, W = plain.load_folder(folder)
        prompts = helpers.random_prompts(pcfg.vocab, [290, 203], 6)
        refs = [plain.forward(pcfg, W, p, torch.bfloat16, windows=WINDOWS) for p in prompts]
        eng = Engine.load(folder, dtype="bfloat16", max_context=512, max_seqs=2, max_tokens=1024, graphs=True)
        win = [g for g in eng.cache.paged_groups if g.window]
        slots = [eng.new_sequence() for _ in prompts]
        eng.step([(s, p[:3]) for s, p in zip(slots, prompts)])
        for t in range(3, 203):
            poison_free_pages(eng)
            out = eng.step([(s, [p[t]]) for s, p in zip(slots, prompts)]).cpu()
            for i, ref in enumerate(refs):
                assert float((out[i] - ref[t]).abs().max()) <= helpers.bf16_logit_tolerance(ref), (t, i)
            assert all(g.pages.held <= 2 * (-(-(g.window - 1) // 64) + 3) for g in win)
