"""Sampling settings, with AntoineBut/TileInfer.jl's names and meanings
(src/engine/sampler.jl:10-25): ``temperature = 0`` is greedy decoding; ``top_k = 0`` and
``top_p = 1`` switch those filters off."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0

    def __post_init__(self):
        if not self.temperature >= 0:
            raise ValueError("temperature must be >= 0")
        if not self.top_k >= 0:
            raise ValueError("top_k must be >= 0")
        if not 0 < self.top_p <= 1:
            raise ValueError("top_p must be in (0, 1]")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0


def mix32(x: int) -> int:
    """lowbias32, the bijective 32-bit mix of src/engine/sampler.jl:34-38."""
    x &= 0xFFFFFFFF
    x = ((x ^ (x >> 16)) * 0x7FEB352D) & 0xFFFFFFFF
    x = ((x ^ (x >> 15)) * 0x846CA68B) & 0xFFFFFFFF
    return x ^ (x >> 16)


def sequence_seed(seed: int, index: int) -> int:
    """The seed of request ``index`` of a generation seeded with ``seed``: a request's tokens do not
    depend on which batch it ran in."""
    return mix32((seed & 0xFFFFFFFF) ^ mix32((index + 0x9E3779B9) & 0xFFFFFFFF))
