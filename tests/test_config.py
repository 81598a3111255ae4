"""Configuration and registry (the style of the reference's test/hub/config.jl:36-90)."""
import json
import os

import pytest

import helpers
from tileinfer_b200.config import (ApertusConfig, ConfigError, config_from_dict, load_config, register_architecture,
                                   registered_architectures, resolve_architecture)


def test_apertus_flat_config_is_read_from_its_keys():
    c = ApertusConfig.from_dict(helpers.TINY_B)
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads) == (3, 96, 6, 3)
    assert c.head_dim == 32 and c.num_attention_heads * c.head_dim != c.hidden_size
    assert c.rope_theta == 12e6 and c.rope_scaling.factor == 8.0
    assert c.rope_scaling.original_max_position_embeddings == 64
    assert c.rms_norm_eps == 1e-6 and c.tie_word_embeddings and c.qk_norm
    assert c.eos_token_ids == (3, 5)
    assert ApertusConfig.from_dict(helpers.TINY_A).eos_token_ids == (7,)
    assert ApertusConfig.from_dict(helpers.TINY_C).eos_token_ids == ()


def test_defaults_and_derived_sizes():
    d = dict(helpers.TINY_A)
    del d["head_dim"], d["num_key_value_heads"]
    c = ApertusConfig.from_dict(d)
    assert c.head_dim == 16 and c.num_key_value_heads == 4
    assert c.dtype == "bfloat16"
    d["rope_parameters"] = {"rope_type": "llama3", "rope_theta": 5e5, "factor": 2.0, "low_freq_factor": 1.0,
                            "high_freq_factor": 4.0, "original_max_position_embeddings": 128}
    c = ApertusConfig.from_dict(d)
    assert c.rope_theta == 5e5 and c.rope_scaling.factor == 2.0
    # Keys a config may leave out take the reference's defaults (src/config.jl:84-91): no q/k norm unless it says
    # so, untied head, no stop tokens.
    for key in ("qk_norm", "tie_word_embeddings", "eos_token_id"):
        d.pop(key, None)
    c = ApertusConfig.from_dict(d)
    assert not c.qk_norm and not c.tie_word_embeddings and c.eos_token_ids == ()
    from tileinfer_b200.engine.model import tensor_declarations
    assert not any("q_norm" in t.name for t in tensor_declarations(c.model_spec()))


def test_round_trip_through_config_json():
    for d in (helpers.TINY_A, helpers.TINY_B, helpers.TINY_C):
        c = ApertusConfig.from_dict(d)
        assert ApertusConfig.from_dict(c.to_dict()) == c


@pytest.mark.parametrize("change, text", [
    ({"post_norm": True}, "post-norm"),
    ({"attention_bias": True}, "attention bias"),
    ({"mlp_bias": True}, "MLP bias"),
    ({"hidden_act": "silu"}, "hidden_act"),
    ({"use_sliding_window": True, "sliding_window": 128}, "sliding-window"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "RoPE scaling"),
    ({"dtype": "int8"}, "dtype"),
    ({"num_key_value_heads": 3}, "multiple"),
])
def test_rejections_name_the_option(change, text):
    with pytest.raises(ConfigError, match=text):
        ApertusConfig.from_dict({**helpers.TINY_A, **change})


def test_missing_key_is_named():
    d = dict(helpers.TINY_A)
    del d["rms_norm_eps"]
    with pytest.raises(ConfigError, match="rms_norm_eps"):
        ApertusConfig.from_dict(d)


def test_registry_resolves_by_architecture_then_model_type():
    assert resolve_architecture(helpers.TINY_A).config_class is ApertusConfig
    assert resolve_architecture({"model_type": "apertus"}).config_class is ApertusConfig
    with pytest.raises(ConfigError, match="ApertusForCausalLM"):
        resolve_architecture({"architectures": ["LlamaForCausalLM"], "model_type": "llama"})
    assert isinstance(config_from_dict(helpers.TINY_A), ApertusConfig)


def test_registering_another_architecture():
    class Other:
        @classmethod
        def from_dict(cls, c):
            return cls()
    register_architecture("OtherForCausalLM", Other, model_type="other")
    assert "OtherForCausalLM" in registered_architectures()
    assert isinstance(config_from_dict({"architectures": ["OtherForCausalLM"]}), Other)


def test_load_config_from_folder(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(helpers.TINY_A))
    assert load_config(str(tmp_path)).hidden_size == 64
    with pytest.raises(ConfigError, match="config.json"):
        load_config(str(tmp_path / "nothing"))


def test_model_spec_lists_layers_and_order():
    spec = ApertusConfig.from_dict(helpers.TINY_B).model_spec()
    assert len(spec.layers) == 3 and spec.order == (0, 1, 2)
    assert spec.lm_head_name is None            # tied
    l = spec.layers[1]
    assert l.mixer.kind == "attention" and l.feed_forward.kind == "xielu_mlp" and l.block == "pre_norm"
    assert l.mixer.position.kind == "rope" and l.mixer.position.scaling.factor == 8.0
    assert abs(l.mixer.scale - 32 ** -0.5) < 1e-12
    assert l.mixer_norm.weight_name == "model.layers.1.attention_layernorm.weight"
