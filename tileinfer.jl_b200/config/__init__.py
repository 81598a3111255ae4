from .apertus import ApertusConfig, ConfigError, parse_rope_scaling
from .registry import (Architecture, config_from_dict, load_config, register_architecture,
                       registered_architectures, resolve_architecture)
from .spec import (FeedForwardSpec, LayerSpec, Llama3RopeScaling, MixerSpec, ModelSpec, NormSpec, PositionSpec,
                   TensorDecl)
