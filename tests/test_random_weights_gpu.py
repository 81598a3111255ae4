"""The random-weights generator on the device against its host form, and the models both make."""
import os
import tempfile

import numpy as np
import pytest
import torch

import helpers
import plain_apertus as plain

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_device_and_host_draw_the_same_bits(dtype):
    """Every init kind, both element types, a count that no block size divides, tensors of a few million
    elements (all octants, both branches of the mantissa fold), and a part of a tensor made alone."""
    from tileinfer_b200.config.spec import TensorDecl
    from tileinfer_b200.kernels import ops
    from tileinfer_b200.weights import random_tensors
    from tileinfer_b200.weights.random_init import standard_normal, tensor_keys
    decls = [TensorDecl("a.weight", (1031, 2053), ("normal", 0.02)), TensorDecl("b.norm", (4099,), ("one_plus_normal", 0.02)),
             TensorDecl("c.alpha", (1,), ("const_plus_normal", 0.2, 0.05)), TensorDecl("d.beta", (), ("const", 0.5)),
             TensorDecl("e.eps", (), ("const", -1e-6)), TensorDecl("f", (3, 5, 7), ("normal", 1.0))]
    host = random_tensors(decls, 17, dtype=dtype, device="cpu")
    dev = random_tensors(decls, 17, dtype=dtype, device="cuda")
    for d in decls:
        assert dev[d.name].is_cuda and dev[d.name].dtype == dtype and tuple(dev[d.name].shape) == tuple(d.shape)
        assert torch.equal(dev[d.name].cpu(), host[d.name]), d.name
    k0, k1 = tensor_keys(17, "a.weight")
    part = torch.empty(1000, dtype=torch.float32, device="cuda")
    ops.random_normal(part, k0, k1, 0.0, 1.0, first=(1 << 32) - 1000)              # the end of the 32-bit counter
    assert np.array_equal(part.cpu().numpy(), standard_normal(k0, k1, (1 << 32) - 1000, 1000))
    z = torch.empty(1 << 22, dtype=torch.float32, device="cuda")
    ops.random_normal(z, k0, k1, 0.0, 1.0)
    assert abs(float(z.mean())) < 2e-3 and abs(float(z.std()) - 1) < 2e-3 and abs(float((z ** 4).mean()) - 3) < 0.02


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_random_engine_is_the_folder_loaded_back_and_the_plain_restatement(dtype):
    """Engine.random(config, seed) draws on the device; write_model_folder draws on the host here; the plain
    implementation restates the generator: one model, the same logits bit for bit from both engines, and
    the plain implementation's within the usual bound."""
    import tileinfer_b200 as ti
    from tileinfer_b200.config import ApertusConfig
    from tileinfer_b200.weights import write_model_folder
    for cfg_dict, seed in ((helpers.TINY_B, 5), (helpers.TINY_D, 6)):
        cfg = ApertusConfig.from_dict(cfg_dict)
        prompts = helpers.random_prompts(cfg.vocab_size, [40, 7], 8)
        with tempfile.TemporaryDirectory() as d:
            folder = write_model_folder(cfg, seed, os.path.join(d, "m"), device="cpu")
            outs = []
            for eng in (ti.Engine.random(cfg, seed, dtype=dtype, max_context=64, max_seqs=2),
                        ti.Engine.load(folder, dtype=dtype, max_context=64, max_seqs=2)):
                slots = [eng.new_sequence() for _ in prompts]
                outs.append(eng.step(list(zip(slots, prompts)), [list(range(len(p))) for p in prompts]).cpu())
            assert torch.equal(outs[0], outs[1])
            pc, _ = plain.load_folder(folder)
        pdt = torch.float32 if dtype == "float32" else torch.bfloat16
        ref = torch.cat([plain.forward(pc, plain.random_weights(pc, seed), p, pdt) for p in prompts])
        scale = float(ref.abs().max())
        assert float((outs[0] - ref).abs().max()) <= (2e-5 * max(scale, 1.0) if dtype == "float32" else 4 * scale * 2.0 ** -8)


def test_a_float16_checkpoint_is_widened_exactly_in_32_bit():
    """A checkpoint stored in float16 runs the 32-bit path on exactly those values (not on values rounded to
    bfloat16 on the way, which loses three bits of each weight and would miss the bound below)."""
    import tileinfer_b200 as ti
    from safetensors.torch import load_file, save_file
    from tileinfer_b200.config import ApertusConfig
    from tileinfer_b200.weights import write_model_folder
    cfg = ApertusConfig.from_dict(helpers.TINY_A)
    with tempfile.TemporaryDirectory() as d:
        folder = write_model_folder(cfg, 9, os.path.join(d, "m"), dtype=torch.float32)
        path = os.path.join(folder, "model.safetensors")
        save_file({k: v.to(torch.float16) for k, v in load_file(path).items()}, path)
        pc, pw = plain.load_folder(folder)                                       # widens float16 to 32-bit
        prompt = helpers.random_prompts(pc.vocab, [50], 2)[0]
        ref = plain.forward(pc, pw, prompt, torch.float32)
        coarse = plain.forward(pc, {k: v.to(torch.bfloat16).float() for k, v in pw.items()}, prompt, torch.float32)
        eng = ti.Engine.load(folder, dtype="float32", max_context=64, max_seqs=1)
        got = eng.step([(eng.new_sequence(), prompt)], [list(range(50))]).cpu()
        tol = 2e-5 * max(float(ref.abs().max()), 1.0)
        assert float((got - ref).abs().max()) <= tol
        assert float((coarse - ref).abs().max()) > 10 * tol                      # the test can tell the two apart
