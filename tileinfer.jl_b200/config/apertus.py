"""Typed configuration of Apertus (``ApertusForCausalLM``), read from its config.json keys.

Apertus is a pre-norm decoder: RMSNorm (``attention_layernorm`` / ``feedforward_layernorm``),
grouped-query attention with a per-head RMSNorm on q and k before llama3-scaled RoPE, and
a non-gated ``up_proj -> xIELU -> down_proj`` feed-forward with four learned scalars per
layer. Keys, defaults and rejections follow the reference's parser
(src/config.jl:48-106); tensor names follow its loader (src/hub/loader.jl:148-202).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .spec import (FeedForwardSpec, LayerSpec, Llama3RopeScaling, MixerSpec, ModelSpec, NormSpec,
                   PositionSpec)

CHECKPOINT_DTYPES = ("bfloat16", "float16", "float32")


class ConfigError(ValueError):
    """A config.json that this library cannot run; the message names the key."""


def _require(c: Mapping[str, Any], key: str) -> Any:
    if key not in c or c[key] is None:
        raise ConfigError(f"config.json has no \"{key}\"")
    return c[key]


def parse_rope_scaling(s: Optional[Mapping[str, Any]]) -> Optional[Llama3RopeScaling]:
    """src/config.jl:99-106: ``default`` means none, ``llama3`` is read, anything else is refused."""
    if s is None:
        return None
    kind = s.get("rope_type", s.get("type", "default"))
    if kind == "default":
        return None
    if kind != "llama3":
        raise ConfigError(f"unsupported RoPE scaling \"{kind}\" (supported: default, llama3)")
    return Llama3RopeScaling(
        factor=float(_require(s, "factor")),
        low_freq_factor=float(_require(s, "low_freq_factor")),
        high_freq_factor=float(_require(s, "high_freq_factor")),
        original_max_position_embeddings=int(_require(s, "original_max_position_embeddings")),
    )


@dataclass(frozen=True)
class ApertusConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: Optional[Llama3RopeScaling]
    max_position_embeddings: int
    tie_word_embeddings: bool
    qk_norm: bool
    hidden_act: str
    dtype: str
    bos_token_id: Optional[int]
    eos_token_ids: Tuple[int, ...]
    initializer_range: float

    architecture = "ApertusForCausalLM"
    model_type = "apertus"

    @classmethod
    def from_dict(cls, c: Mapping[str, Any]) -> "ApertusConfig":
        hidden_act = c.get("hidden_act", "xielu")
        if hidden_act != "xielu":
            raise ConfigError(f"unsupported hidden_act \"{hidden_act}\" for Apertus (expected \"xielu\")")
        if c.get("post_norm", False):
            raise ConfigError("Apertus post-norm layers (post_norm: true) are not supported")
        if c.get("use_sliding_window", False) and c.get("sliding_window") is not None:
            raise ConfigError("sliding-window attention (use_sliding_window) is not part of Apertus")
        if c.get("attention_bias", False):
            raise ConfigError("attention biases (attention_bias: true) are not supported")
        if c.get("mlp_bias", False):
            raise ConfigError("MLP biases (mlp_bias: true) are not supported")

        # transformers >= 5 nests the RoPE settings under rope_parameters (src/config.jl:66-69).
        rope = c.get("rope_parameters")
        if rope is None:
            rope_theta = _require(c, "rope_theta")
            scaling = c.get("rope_scaling")
        else:
            rope_theta = _require(rope, "rope_theta")
            scaling = rope
        heads = int(_require(c, "num_attention_heads"))
        hidden = int(_require(c, "hidden_size"))
        head_dim = c.get("head_dim")
        if head_dim is None:
            if hidden % heads:
                raise ConfigError(f"hidden_size {hidden} is not a multiple of num_attention_heads {heads} "
                                  "and config.json gives no head_dim")
            head_dim = hidden // heads
        kv_heads = int(c.get("num_key_value_heads") or heads)
        if heads % kv_heads:
            raise ConfigError(f"num_attention_heads {heads} is not a multiple of num_key_value_heads {kv_heads}")
        if int(head_dim) % 2:
            raise ConfigError(f"head_dim {head_dim} must be even for rotary embeddings")
        dtype = c.get("dtype", c.get("torch_dtype", "bfloat16"))
        if dtype not in CHECKPOINT_DTYPES:
            raise ConfigError(f"unsupported checkpoint dtype \"{dtype}\" (supported: {', '.join(CHECKPOINT_DTYPES)})")
        eos = c.get("eos_token_id")
        eos_ids = () if eos is None else (int(eos),) if isinstance(eos, int) else tuple(int(e) for e in eos)
        return cls(
            vocab_size=int(c.get("output_vocab_size") or _require(c, "vocab_size")),
            hidden_size=hidden,
            intermediate_size=int(_require(c, "intermediate_size")),
            num_hidden_layers=int(_require(c, "num_hidden_layers")),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=int(head_dim),
            rms_norm_eps=float(_require(c, "rms_norm_eps")),
            rope_theta=float(rope_theta),
            rope_scaling=parse_rope_scaling(scaling),
            max_position_embeddings=int(_require(c, "max_position_embeddings")),
            tie_word_embeddings=bool(c.get("tie_word_embeddings", False)),
            # Apertus checkpoints say qk_norm: true; a config without the key has none, as in the reference
            # (src/config.jl:91: the default is false for every model type but qwen3).
            qk_norm=bool(c.get("qk_norm", False)),
            hidden_act=hidden_act,
            dtype=dtype,
            bos_token_id=c.get("bos_token_id"),
            eos_token_ids=eos_ids,
            initializer_range=float(c.get("initializer_range", 0.02)),
        )

    def to_dict(self) -> dict:
        """The config.json that :meth:`from_dict` reads back to this configuration."""
        d = {
            "architectures": [self.architecture],
            "model_type": self.model_type,
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "qk_norm": self.qk_norm,
            "hidden_act": self.hidden_act,
            "attention_bias": False,
            "mlp_bias": False,
            "dtype": self.dtype,
            "initializer_range": self.initializer_range,
        }
        if self.rope_scaling is not None:
            s = self.rope_scaling
            d["rope_scaling"] = {
                "rope_type": "llama3", "factor": s.factor, "low_freq_factor": s.low_freq_factor,
                "high_freq_factor": s.high_freq_factor,
                "original_max_position_embeddings": s.original_max_position_embeddings,
            }
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    def model_spec(self) -> ModelSpec:
        """Lower to the per-layer records the engine builds parts from."""
        H, D = self.hidden_size, self.head_dim
        position = PositionSpec(kind="rope", head_dim=D, theta=self.rope_theta, scaling=self.rope_scaling,
                                max_positions=self.max_position_embeddings)
        # Raw xIELU parameters of the random-weights mode: softplus(raw) = 0.8.
        raw_alpha = math.log(math.expm1(0.8))
        layers = []
        for l in range(self.num_hidden_layers):
            p = f"model.layers.{l}."
            mixer = MixerSpec(
                kind="attention", prefix=p + "self_attn.", hidden_size=H,
                num_heads=self.num_attention_heads, num_kv_heads=self.num_key_value_heads, head_dim=D,
                qk_norm=self.qk_norm, qk_norm_eps=self.rms_norm_eps,
                # The reference fixes the softmax scale to 1/sqrt(head_dim) (src/model/decoder.jl:169).
                scale=1.0 / math.sqrt(D), position=position,
                tensor_names={"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight",
                              "o": "o_proj.weight", "q_norm": "q_norm.weight", "k_norm": "k_norm.weight"},
                options={"init_std": self.initializer_range},
            )
            ffn = FeedForwardSpec(
                kind="xielu_mlp", prefix=p + "mlp.", hidden_size=H, intermediate_size=self.intermediate_size,
                tensor_names={"up": "up_proj.weight", "down": "down_proj.weight",
                              "alpha_p": "act_fn.alpha_p", "alpha_n": "act_fn.alpha_n",
                              "beta": "act_fn.beta", "eps": "act_fn.eps"},
                options={"init_std": self.initializer_range, "init_alpha_raw": raw_alpha,
                         "init_alpha_std": 0.05, "init_beta": 0.5, "init_eps": -1e-6},
            )
            layers.append(LayerSpec(
                block="pre_norm", mixer=mixer,
                mixer_norm=NormSpec("rmsnorm", H, self.rms_norm_eps, p + "attention_layernorm.weight",
                                    {"init_std": self.initializer_range}),
                feed_forward=ffn,
                feed_forward_norm=NormSpec("rmsnorm", H, self.rms_norm_eps, p + "feedforward_layernorm.weight",
                                           {"init_std": self.initializer_range}),
            ))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab_size, hidden_size=H,
            layers=tuple(layers), order=tuple(range(self.num_hidden_layers)),
            final_norm=NormSpec("rmsnorm", H, self.rms_norm_eps, "model.norm.weight",
                                {"init_std": self.initializer_range}),
            embed_name="model.embed_tokens.weight",
            lm_head_name=None if self.tie_word_embeddings else "lm_head.weight",
            max_positions=self.max_position_embeddings,
            eos_token_ids=self.eos_token_ids, bos_token_id=self.bos_token_id,
            init_std=self.initializer_range,
        )
