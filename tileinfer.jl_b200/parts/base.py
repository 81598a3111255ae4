"""Interfaces of the parts a layer is put together from, and their registries.

A layer is a *block* (the arrangement) around a *mixer* (attention here), a *feed-forward*
and two *norms*; a mixer may apply a *position encoding*. Each part is built from its own
record of sizes and constants (``config.spec``), the tensors it declared, and the runtime;
it never sees the model's configuration. Parts are looked up by the ``kind`` string of
their record, so a new kind is added by registering a class here, from anywhere.

Interfaces (duck-typed; the base classes document them):

* ``Norm(spec, tensors, rt)``: ``forward(x, out)``; ``add_forward(x, delta, out)`` does
  ``x += delta`` then ``out = norm(x)`` in one kernel (``delta`` may be 32-bit partial sums [s, n, size]).
* ``PositionEncoding(spec, rt, max_positions)``: ``rotation()`` returns the :class:`Rotation` that the
  attention mixer applies to queries and keys (a table of cos/sin per position and pair, how many
  elements of a head it covers, and which elements are paired), or None for an encoding that rotates
  nothing; an encoding of another kind offers methods of its own to the mixers written for it.
* ``Mixer(spec, tensors, rt, position)``: ``cache_request()`` says what per-sequence storage a
  layer of this kind needs; ``forward(h, step, cache) -> delta`` mixes tokens of the same
  sequence, reading and writing ``cache`` (the layer's view of its cache group);
  ``decode_plan(group)`` may ask for tables of its own in the metadata of one-token steps.
* ``FeedForward(spec, tensors, rt)``: ``forward(h, step) -> delta``, token by token.
* ``Block(layer_spec, mixer, feed_forward, mixer_norm, feed_forward_norm)``:
  ``forward(x, h, step, cache, next_norm, h_out)``.
* ``Embedding(model_spec, tensors, rt)`` and ``Head(model_spec, tensors, rt, embedding)``: the two ends of the
  model (``ModelSpec.embedding_kind`` / ``head_kind``), so that an embedding multiplier or a scaled or capped
  logit is a registered part, not an edit of the decoder.

Every class also has ``tensors(spec) -> [TensorDecl]``: the checkpoint tensors it reads,
with shapes, used by the loader's checks and by the random-weights mode.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch

from ..config.spec import TensorDecl


@dataclass(frozen=True)
class CacheRequest:
    """Per-sequence storage a mixer needs for one layer.

    ``kind == "paged_kv"``: keys and values of every position (or of the last ``window``),
    ``kv_heads × head_dim`` each, in pages. ``kind == "state"``: a tensor of fixed ``shape``
    and ``dtype`` per sequence, zeroed when a sequence starts. Any other kind is one that was
    registered with ``cache.register_cache_kind``; its group class reads what it needs from these fields.
    """
    kind: str
    kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    shape: Tuple[int, ...] = ()
    dtype: Optional[torch.dtype] = None          # None: the model's element type

    def group_key(self):
        return (self.kind, self.kv_heads, self.head_dim, self.window, tuple(self.shape), self.dtype)


class Part:
    @classmethod
    def tensors(cls, spec) -> List[TensorDecl]:
        return []


class Norm(Part):
    def forward(self, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def add_forward(self, x, delta, out):
        raise NotImplementedError


@dataclass(frozen=True)
class Rotation:
    """A rotation of pairs of a head's elements by angles that depend on the position, as the
    attention-inputs kernel applies it to queries and keys after their norm.

    ``cos_sin``: float32 ``[max_positions, rotary_dim / 2, 2]`` holding (cos, sin) of every (position,
    pair), already rounded to the model's element type. ``rotary_dim`` (even, at most the head size): the
    first so many elements of a head are rotated, the rest pass through. ``interleaved`` False: element i
    pairs with i + rotary_dim / 2 (rotate-half, what Apertus uses: AntoineBut/TileInfer.jl
    src/ops/interface.jl:46-52); True: element 2i pairs with 2i + 1.
    """
    cos_sin: torch.Tensor
    rotary_dim: int
    interleaved: bool = False


class PositionEncoding(Part):
    def rotation(self) -> Optional[Rotation]:
        """What an attention mixer applies to q and k; None: nothing."""
        return None


class Mixer(Part):
    def cache_request(self) -> Optional[CacheRequest]:
        return None

    def decode_plan(self, group) -> Optional[Any]:
        """Tables that this mixer's kernels want in the metadata of one-token steps, beside what every step
        carries, or None. ``group`` is the cache group of the mixer's layers (the first mixer of a group is
        asked, once). The returned object's ``native`` field is a C++ ``ti::GroupPlan`` (``csrc/host/host_common.h``:
        how many words a step of a given batch size needs, and how to fill them from the sequences' lengths);
        the step planner reserves and fills those words every step and hands them to the mixer as
        ``step.group(i).plan_table``, with the object itself as ``step.group(i).plan``."""
        return None

    def forward(self, h: torch.Tensor, step, cache) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, h: torch.Tensor, step) -> torch.Tensor:
        raise NotImplementedError


class Embedding(Part):
    """Token ids to the residual stream. ``__init__(spec: ModelSpec, tensors, rt)``; ``table`` is the matrix a tied
    head shares; ``forward(token_ids, out, status)`` writes ``out`` [n, hidden] (``status``: a device word that
    receives 1 + the index of a token whose id is outside the vocabulary)."""

    def forward(self, token_ids: torch.Tensor, out: torch.Tensor, status: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Head(Part):
    """The final norm's output at the wanted rows to 32-bit logits. ``__init__(spec: ModelSpec, tensors, rt,
    embedding)`` (the embedding part, whose table a tied head uses); ``forward(h, logits)``."""

    def forward(self, h: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


_REGISTRIES: Dict[str, Dict[str, Any]] = {"mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "block": {},
                                          "embedding": {}, "head": {}}


def _register(family: str, kind: str, cls):
    _REGISTRIES[family][kind] = cls
    return cls


def register_mixer(kind: str, cls=None):
    return _register("mixer", kind, cls) if cls is not None else (lambda c: _register("mixer", kind, c))


def register_feed_forward(kind: str, cls=None):
    return _register("feed_forward", kind, cls) if cls is not None else (lambda c: _register("feed_forward", kind, c))


def register_norm(kind: str, cls=None):
    return _register("norm", kind, cls) if cls is not None else (lambda c: _register("norm", kind, c))


def register_position(kind: str, cls=None):
    return _register("position", kind, cls) if cls is not None else (lambda c: _register("position", kind, c))


def register_block(kind: str, cls=None):
    return _register("block", kind, cls) if cls is not None else (lambda c: _register("block", kind, c))


def register_embedding(kind: str, cls=None):
    return _register("embedding", kind, cls) if cls is not None else (lambda c: _register("embedding", kind, c))


def register_head(kind: str, cls=None):
    return _register("head", kind, cls) if cls is not None else (lambda c: _register("head", kind, c))


def lookup(family: str, kind: str):
    try:
        return _REGISTRIES[family][kind]
    except KeyError:
        known = ", ".join(sorted(_REGISTRIES[family])) or "none"
        raise KeyError(f"no {family} part of kind \"{kind}\" is registered (registered: {known})") from None
