"""Weights: reading by name, the one error that lists everything wrong, the random-weights folder."""
import json
import os
import struct

import pytest
import torch

import helpers
from tileinfer_b200.config import ApertusConfig
from tileinfer_b200.engine.model import ignorable_tensors, tensor_declarations
from tileinfer_b200.weights import (SafetensorsError, SafetensorsFile, WeightsError, load_tensors, open_folder,
                                    random_tensors, save_file, write_model_folder)


def _folder(tmp_path, cfg_dict=helpers.TINY_A, seed=0, dtype=torch.bfloat16):
    cfg = ApertusConfig.from_dict(cfg_dict)
    return cfg, write_model_folder(cfg, seed, str(tmp_path / "m"), dtype=dtype)


def test_random_folder_loads_back_and_is_seeded(tmp_path):
    cfg, d = _folder(tmp_path)
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    spec = cfg.model_spec()
    t = load_tensors(d, tensor_declarations(spec))
    again = random_tensors(tensor_declarations(spec), 0)
    other = random_tensors(tensor_declarations(spec), 1)
    for k, v in t.items():
        assert v.dtype == torch.bfloat16
        assert torch.equal(v, again[k])
    assert not torch.equal(t["model.embed_tokens.weight"], other["model.embed_tokens.weight"])
    assert ApertusConfig.from_dict(json.load(open(os.path.join(d, "config.json")))) == cfg


def test_random_distributions():
    cfg = ApertusConfig.from_dict(helpers.TINY_B)
    t = random_tensors(tensor_declarations(cfg.model_spec()), 3, dtype=torch.float32)
    w = t["model.layers.0.mlp.up_proj.weight"]
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(w.mean())) < 0.002
    n = t["model.layers.1.attention_layernorm.weight"]
    assert abs(float(n.mean()) - 1.0) < 0.02
    assert float(t["model.layers.0.mlp.act_fn.beta"]) == 0.5
    assert abs(float(t["model.layers.0.mlp.act_fn.eps"]) + 1e-6) < 1e-9
    a = float(t["model.layers.2.mlp.act_fn.alpha_p"])
    assert abs(torch.nn.functional.softplus(torch.tensor(a)) - 0.8) < 0.2
    assert "lm_head.weight" not in t            # tied


def test_the_generator_is_a_function_of_seed_name_and_index():
    """value = f(seed, tensor name, element index): a part of a tensor can be made alone, other tensors
    change nothing, and the plain implementation's restatement of the function gives the same bits."""
    import numpy as np
    import plain_apertus as plain
    from tileinfer_b200.config.spec import TensorDecl
    from tileinfer_b200.weights.random_init import standard_normal, tensor_keys
    name = "model.layers.3.mlp.down_proj.weight"
    k0, k1 = tensor_keys(5, name)
    z = standard_normal(k0, k1, 0, 70000)
    assert z.dtype == np.float32 and np.array_equal(z[1234:1300], standard_normal(k0, k1, 1234, 66))
    assert np.array_equal(z, plain.random_normal(5, name, 70000))
    # Near the end of the 32-bit counter, and refused beyond it.
    assert standard_normal(k0, k1, (1 << 32) - 8, 8).shape == (8,)
    with pytest.raises(ValueError, match="32-bit counter"):
        standard_normal(k0, k1, (1 << 32) - 8, 9)
    assert abs(float(z.mean())) < 0.02 and abs(float(z.std()) - 1) < 0.02 and abs(float((z ** 4).mean()) - 3) < 0.2
    assert tensor_keys(5, name) != tensor_keys(6, name) and tensor_keys(5, name) != tensor_keys(5, name + "x")
    alone = random_tensors([TensorDecl(name, (7, 9), ("normal", 0.02))], 5)[name]
    among = random_tensors([TensorDecl("other", (3,), ("normal", 1.0)), TensorDecl(name, (7, 9), ("normal", 0.02))], 5)[name]
    assert torch.equal(alone, among)
    want = torch.from_numpy(np.float32(0.0) + z[:63] * np.float32(0.02)).to(torch.bfloat16).view(7, 9)
    assert torch.equal(alone, want)


def test_the_plain_implementation_regenerates_a_random_model(tmp_path):
    """Folder written by the library == weights restated by the plain implementation, tensor by tensor."""
    import plain_apertus as plain
    for cfg_dict, seed in ((helpers.TINY_A, 0), (helpers.TINY_B, 1), (helpers.TINY_C, 2)):
        cfg, d = _folder(tmp_path / str(seed), cfg_dict, seed)
        pc, stored = plain.load_folder(d)
        again = plain.random_weights(pc, seed)
        assert set(again) == set(stored)
        for k in stored:
            assert torch.equal(stored[k].reshape(-1), again[k].reshape(-1)), k


def test_stored_types_are_kept(tmp_path):
    tensors = {"a": torch.randn(3, 4).to(torch.bfloat16), "b": torch.randn(3), "c": torch.arange(5),
               "d": torch.randn(2, 2).to(torch.float16)}
    os.makedirs(tmp_path / "m")
    save_file(tensors, str(tmp_path / "m" / "model.safetensors"))
    from tileinfer_b200.config.spec import TensorDecl
    decls = [TensorDecl("a", (3, 4), ("normal", 1)), TensorDecl("b", (3,), ("normal", 1)),
             TensorDecl("c", (5,), ("normal", 1)), TensorDecl("d", (2, 2), ("normal", 1))]
    t = load_tensors(str(tmp_path / "m"), decls)
    assert t["a"].dtype == torch.bfloat16 and torch.equal(t["a"], tensors["a"])
    assert t["b"].dtype == torch.float32 and torch.equal(t["b"], tensors["b"])
    assert t["c"].dtype == torch.int32 and t["c"].tolist() == [0, 1, 2, 3, 4]
    # float16 is kept as stored: the 32-bit path widens it exactly, a bfloat16 run rounds it once.
    assert t["d"].dtype == torch.float16 and torch.equal(t["d"], tensors["d"])


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg, d = _folder(tmp_path)
    by_name, _ = open_folder(d)
    tensors = {k: f.tensor(k).clone() for k, f in by_name.items()}
    del tensors["model.layers.0.self_attn.q_norm.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.mlp.gate_proj.weight"] = torch.zeros(2, 2)
    tensors["model.layers.1.mlp.up_proj.weight"] = torch.zeros(10, 64, dtype=torch.bfloat16)
    save_file(tensors, os.path.join(d, "model.safetensors"))
    with pytest.raises(WeightsError) as e:
        load_tensors(d, tensor_declarations(cfg.model_spec()))
    err = e.value
    assert set(err.missing) == {"model.layers.0.self_attn.q_norm.weight", "model.norm.weight"}
    assert err.unexpected == ["model.layers.0.mlp.gate_proj.weight"]
    assert err.wrong_shape == [("model.layers.1.mlp.up_proj.weight", (10, 64), (192, 64))]
    text = str(err)
    for needle in ("missing tensors (2)", "q_norm", "unexpected tensors (1)", "gate_proj", "wrong shapes (1)",
                   "[10, 64], expected [192, 64]"):
        assert needle in text


def test_tied_checkpoint_may_keep_a_head_copy_and_padded_embedding(tmp_path):
    cfg, d = _folder(tmp_path, helpers.TINY_B)
    spec = cfg.model_spec()
    by_name, _ = open_folder(d)
    tensors = {k: f.tensor(k).clone() for k, f in by_name.items()}
    tensors["lm_head.weight"] = torch.zeros(512, 96, dtype=torch.bfloat16)
    tensors["model.embed_tokens.weight"] = torch.cat([tensors["model.embed_tokens.weight"],
                                                      torch.ones(64, 96, dtype=torch.bfloat16)])
    save_file(tensors, os.path.join(d, "model.safetensors"))
    t = load_tensors(d, tensor_declarations(spec), ignorable_tensors(spec))
    assert t["model.embed_tokens.weight"].shape == (512, 96)
    with pytest.raises(WeightsError, match="unexpected"):
        load_tensors(d, tensor_declarations(spec))


def test_container_errors(tmp_path):
    os.makedirs(tmp_path / "e")
    with pytest.raises(SafetensorsError, match="no .safetensors"):
        open_folder(str(tmp_path / "e"))
    p = tmp_path / "e" / "model.safetensors"
    save_file({"x": torch.randn(8, 8)}, str(p))
    raw = p.read_bytes()
    p.write_bytes(raw[:-16])
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 10) + b"not json!!")
    with pytest.raises(SafetensorsError, match="JSON"):
        SafetensorsFile(str(p))
    save_file({"x": torch.randn(2)}, str(p))
    save_file({"x": torch.randn(2)}, str(tmp_path / "e" / "other.safetensors"))
    with pytest.raises(SafetensorsError, match="twice"):
        open_folder(str(tmp_path / "e"))


def test_reads_files_written_by_the_safetensors_package(tmp_path):
    from safetensors.torch import save_file as st_save
    tensors = {"w": torch.randn(5, 7).to(torch.bfloat16), "s": torch.tensor(0.5)}
    st_save(tensors, str(tmp_path / "model.safetensors"))
    f = SafetensorsFile(str(tmp_path / "model.safetensors"))
    assert torch.equal(f.tensor("w"), tensors["w"]) and float(f.tensor("s")) == 0.5
    from safetensors import safe_open
    save_file(tensors, str(tmp_path / "ours.safetensors"))
    with safe_open(str(tmp_path / "ours.safetensors"), "pt") as g:
        assert torch.equal(g.get_tensor("w"), tensors["w"]) and g.get_tensor("s").shape == ()


def test_weight_bytes_counts_what_a_step_reads():
    """Every matrix and norm vector once, the head included, a tied head once, the embedding table of an
    untied model not at all (a step reads one row per token); this is the roofline's weight term."""
    from tileinfer_b200.engine.model import DecoderModel
    from tileinfer_b200.parts import Runtime
    for cfg_dict in (helpers.TINY_A, helpers.TINY_B):
        cfg = ApertusConfig.from_dict(cfg_dict)
        spec = cfg.model_spec()
        tensors = random_tensors(tensor_declarations(spec), 0)
        model = DecoderModel(spec, tensors, Runtime(torch.bfloat16, "cpu"), 64)
        read = {k: v for k, v in tensors.items() if v.numel() > 1 and (k != "model.embed_tokens.weight" or cfg.tie_word_embeddings)}
        assert ("lm_head.weight" in read) == (not cfg.tie_word_embeddings)
        assert model.weight_bytes() == sum(v.numel() * 2 for v in read.values())
