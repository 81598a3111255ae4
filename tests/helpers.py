"""Shared by the tests: tiny configurations, the reference fixture, tolerances."""
from __future__ import annotations

import json
import math
import os
import random
import shutil
import tempfile

import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# Two tiny Apertus configurations that differ in every size and option.
TINY_A = {
    "architectures": ["ApertusForCausalLM"], "model_type": "apertus",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 192, "vocab_size": 256, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-5, "qk_norm": True, "tie_word_embeddings": False, "hidden_act": "xielu",
    "max_position_embeddings": 512, "attention_bias": False, "mlp_bias": False, "eos_token_id": 7,
}
TINY_B = {
    "architectures": ["ApertusForCausalLM"], "model_type": "apertus",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 6, "num_key_value_heads": 3,
    "head_dim": 32, "intermediate_size": 320, "vocab_size": 512, "rope_theta": 12000000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "original_max_position_embeddings": 64,
                     "low_freq_factor": 1.0, "high_freq_factor": 4.0},
    "rms_norm_eps": 1e-6, "qk_norm": True, "tie_word_embeddings": True, "hidden_act": "xielu",
    "max_position_embeddings": 1024, "attention_bias": False, "mlp_bias": False, "eos_token_id": [3, 5],
}
# A third one with sizes that are no power of two anywhere and a single KV head.
TINY_C = {
    "architectures": ["ApertusForCausalLM"], "model_type": "apertus",
    "num_hidden_layers": 2, "hidden_size": 120, "num_attention_heads": 5, "num_key_value_heads": 1,
    "head_dim": 48, "intermediate_size": 200, "vocab_size": 301, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "original_max_position_embeddings": 32,
                     "low_freq_factor": 1.0, "high_freq_factor": 2.0},
    "rms_norm_eps": 3e-6, "qk_norm": False, "tie_word_embeddings": False, "hidden_act": "xielu",
    "max_position_embeddings": 2048, "attention_bias": False, "mlp_bias": False,
}

# A fourth one with the head size (64) and a group (2) that the tensor-core prefill attention takes, and
# widths that the tensor-core products take, so that replay runs through those kernels too.
TINY_D = {
    "architectures": ["ApertusForCausalLM"], "model_type": "apertus",
    "num_hidden_layers": 2, "hidden_size": 136, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 64, "intermediate_size": 328, "vocab_size": 392, "rope_theta": 1000000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "original_max_position_embeddings": 128,
                     "low_freq_factor": 1.0, "high_freq_factor": 4.0},
    "rms_norm_eps": 2e-6, "qk_norm": True, "tie_word_embeddings": False, "hidden_act": "xielu",
    "max_position_embeddings": 1024, "attention_bias": False, "mlp_bias": False,
}


def reference_fixture_folder(out_dir: str) -> str:
    """The reference's tiny checkpoint, rewritten to the ApertusForCausalLM layout in ``out_dir``:
    flat config, ``model.`` prefix, embedding cut to the text vocabulary (what the reference's loader
    does when reading it: src/config.jl:54-56, 79; src/hub/loader.jl:152-156)."""
    from safetensors import safe_open
    from safetensors.torch import save_file
    src = os.path.join(GOLDEN, "reference_fixture")
    with open(os.path.join(src, "config.json")) as f:
        nested = json.load(f)["text_config"]
    rp = nested["rope_parameters"]
    flat = {k: v for k, v in nested.items() if k not in ("rope_parameters", "output_vocab_size", "model_type")}
    flat.update({"architectures": ["ApertusForCausalLM"], "model_type": "apertus",
                 "vocab_size": nested["output_vocab_size"], "rope_theta": rp["rope_theta"],
                 "rope_scaling": {k: v for k, v in rp.items() if k != "rope_theta"}})
    tensors = {}
    with safe_open(os.path.join(src, "model.safetensors"), "pt") as f:
        for k in f.keys():
            t = f.get_tensor(k)
            name = k.replace("model.language_model.", "model.")
            if name == "model.embed_tokens.weight":
                t = t[: flat["vocab_size"]].contiguous()
            tensors[name] = t
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(flat, f)
    save_file(tensors, os.path.join(out_dir, "model.safetensors"))
    return out_dir


def reference_goldens() -> dict:
    with open(os.path.join(GOLDEN, "reference_fixture", "logits.json")) as f:
        return json.load(f)["cases"]


def random_prompts(vocab: int, lengths, seed: int):
    rng = random.Random(seed)
    return [[rng.randrange(vocab) for _ in range(n)] for n in lengths]


def bf16_logit_tolerance(ref: torch.Tensor) -> float:
    """Absolute tolerance for bfloat16 logits: a few bfloat16 steps at the scale of the logits."""
    scale = float(ref.abs().max())
    return max(8 * scale * 2.0 ** -8, 1e-3)
