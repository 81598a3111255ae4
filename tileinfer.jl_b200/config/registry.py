"""The one registry from an architecture's name to its configuration and model.

``config.json`` names its architecture in ``architectures[0]`` (fallback: ``model_type``);
the entry gives the typed configuration class, whose ``model_spec()`` lowers it to the
per-layer records that :class:`tileinfer_b200.engine.model.DecoderModel` is built from.
The reference keeps a tuple of supported ``model_type`` strings (src/config.jl:8, 52-53).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping, Optional

from .apertus import ApertusConfig, ConfigError


@dataclass(frozen=True)
class Architecture:
    name: str                       # e.g. "ApertusForCausalLM"
    model_type: Optional[str]       # e.g. "apertus"
    config_class: Any               # has from_dict(mapping) and .model_spec()
    # Builds the runnable model from (model_spec, tensors, dtype, device); None selects
    # the library's generic decoder.
    model_factory: Optional[Callable[..., Any]] = None


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_class: Any, model_type: Optional[str] = None,
                          model_factory: Optional[Callable[..., Any]] = None) -> Architecture:
    arch = Architecture(name, model_type, config_class, model_factory)
    _ARCHITECTURES[name] = arch
    return arch


def registered_architectures() -> tuple:
    return tuple(sorted(_ARCHITECTURES))


def resolve_architecture(config: Mapping[str, Any]) -> Architecture:
    names = config.get("architectures") or []
    for n in names:
        if n in _ARCHITECTURES:
            return _ARCHITECTURES[n]
    model_type = config.get("model_type")
    if not names and model_type is not None:
        for arch in _ARCHITECTURES.values():
            if arch.model_type == model_type:
                return arch
    asked = names[0] if names else model_type
    raise ConfigError(f"unsupported architecture \"{asked}\"; supported: {', '.join(registered_architectures())}")


def config_from_dict(config: Mapping[str, Any]):
    """Typed configuration of whichever registered architecture ``config`` names."""
    return resolve_architecture(config).config_class.from_dict(config)


def load_config(model_dir: str):
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{model_dir} has no config.json")
    with open(path) as f:
        return config_from_dict(json.load(f))


register_architecture(ApertusConfig.architecture, ApertusConfig, model_type=ApertusConfig.model_type)
