"""Architecture-neutral description of a model, as the engine consumes it.

An architecture's typed configuration (for instance :class:`ApertusConfig`) is read from
its own ``config.json`` keys and then lowered to a :class:`ModelSpec`: a list of layers,
each naming the kind and the sizes of its mixer, feed-forward, norms and position
encoding, plus the order in which the layers run. Parts are built from these records
alone, so no part knows which model it belongs to, and one model may mix kinds freely.

The reference keeps one flat struct with per-family flags (src/config.jl:24-43) and a
hard-coded layer body (src/model/decoder.jl:165-196); the split into per-layer records is
this library's own.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


@dataclass(frozen=True)
class TensorDecl:
    """One tensor a part expects in the checkpoint.

    ``init`` names the distribution used by the random-weights mode:
    ``("normal", std)``, ``("one_plus_normal", std)``, ``("const_plus_normal", c, std)``
    or ``("const", c)``. ``keep_dtype`` tensors are never cast to the compute dtype (small
    scalars that the part reads on the host in 32-bit).
    """
    name: str
    shape: Tuple[int, ...]
    init: Tuple[Any, ...]
    keep_dtype: bool = False
    # When True the checkpoint may hold more leading rows than ``shape[0]``; the first
    # ``shape[0]`` are used (an embedding table padded beyond the vocabulary).
    allow_extra_rows: bool = False


@dataclass(frozen=True)
class Llama3RopeScaling:
    """Frequency-dependent RoPE scaling (``rope_type == "llama3"``), src/config.jl:11-16."""
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int


@dataclass(frozen=True)
class PositionSpec:
    """Position encoding applied inside a mixer. ``kind`` selects the registered part."""
    kind: str                      # "rope" | "none" | user-registered
    head_dim: int = 0
    theta: float = 10000.0
    scaling: Optional[Llama3RopeScaling] = None
    max_positions: int = 0
    options: Mapping[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class NormSpec:
    kind: str                      # "rmsnorm"
    size: int
    eps: float
    weight_name: str               # checkpoint tensor name (full)
    options: Mapping[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class MixerSpec:
    """Token mixer of a layer.

    For ``kind == "attention"`` the fields below are used; other kinds may keep their own
    sizes in ``options``. ``window`` is the number of most recent keys a query may see
    (None: all). ``kv_source`` is the index (in ``ModelSpec.layers``) of another layer
    whose cached keys and values this layer reads instead of writing its own.
    """
    kind: str
    prefix: str                    # checkpoint name prefix of this mixer's tensors
    hidden_size: int
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    qk_norm: bool = False
    qk_norm_eps: float = 0.0
    scale: float = 0.0             # softmax scale, 1/sqrt(head_dim) where the architecture says so
    window: Optional[int] = None
    kv_source: Optional[int] = None
    position: PositionSpec = PositionSpec(kind="none")
    tensor_names: Mapping[str, str] = field(default_factory=dict)
    options: Mapping[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str                      # "xielu_mlp" | user-registered
    prefix: str
    hidden_size: int
    intermediate_size: int = 0
    tensor_names: Mapping[str, str] = field(default_factory=dict)
    options: Mapping[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    block: str                     # arrangement: "pre_norm"
    mixer: MixerSpec
    mixer_norm: NormSpec
    feed_forward: FeedForwardSpec
    feed_forward_norm: NormSpec


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    layers: Tuple[LayerSpec, ...]
    # Execution order: indices into ``layers``; an index may appear more than once.
    order: Tuple[int, ...]
    final_norm: NormSpec
    embed_name: str
    lm_head_name: Optional[str]    # None: tied to the embedding table
    max_positions: int
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    # Standard deviation of the random-weights mode for matrices.
    init_std: float = 0.02
    # The two ends of the model are parts too, looked up by kind like the layers' parts: how token ids become
    # the residual stream ("lookup": rows of the table, unscaled) and how the final norm's output becomes
    # logits ("linear": a product with the head matrix, 32-bit out). ``options`` is theirs to read.
    embedding_kind: str = "lookup"
    head_kind: str = "linear"
    options: Mapping[str, Any] = field(default_factory=dict)
