"""Rotary position embedding with optional llama3 frequency scaling.

Tables are computed once on the host the way AntoineBut/TileInfer.jl does
(src/model/rope.jl:15-48): inverse frequencies and angles in 32-bit, cos/sin in 64-bit of
the 32-bit angle, rounded to 32-bit and then to the model's element type. The scaling is
static: it does not depend on the running sequence length. The device table is
``[max_positions, rotary_dim/2, 2]`` float32 holding (cos, sin) already rounded to the
element type; both elements of a pair share the angle.

Two options of the record go beyond what Apertus uses: ``rotary_dim`` (rotate only the first so
many elements of a head; default: all) and ``pairing`` ("half": element i with i + rotary_dim/2,
the default; "interleaved": 2i with 2i + 1).
"""
from __future__ import annotations

import math

import torch

from ..config.spec import PositionSpec
from .base import PositionEncoding, Rotation, register_position


def rotary_dim(spec: PositionSpec) -> int:
    D = int(spec.options.get("rotary_dim", spec.head_dim))
    if D < 2 or D % 2 or D > spec.head_dim:
        raise ValueError(f"rotary_dim {D} must be even and between 2 and the head size {spec.head_dim}")
    return D


def inverse_frequencies(spec: PositionSpec) -> torch.Tensor:
    D = rotary_dim(spec)
    theta = torch.tensor(float(spec.theta), dtype=torch.float32)
    inv = 1.0 / (theta ** (torch.arange(0, D, 2, dtype=torch.float32) / torch.tensor(float(D), dtype=torch.float32)))
    s = spec.scaling
    if s is None:
        return inv
    f32 = lambda v: torch.tensor(float(v), dtype=torch.float32)
    factor, low, high = f32(s.factor), f32(s.low_freq_factor), f32(s.high_freq_factor)
    old = f32(s.original_max_position_embeddings)
    wavelen = 2.0 * f32(math.pi) / inv
    smooth = (old / wavelen - low) / (high - low)
    blended = (1 - smooth) * inv / factor + smooth * inv
    return torch.where(wavelen < old / high, inv, torch.where(wavelen > old / low, inv / factor, blended))


@register_position("rope")
class RotaryEmbedding(PositionEncoding):
    def __init__(self, spec: PositionSpec, rt, max_positions: int):
        self.spec = spec
        self.max_positions = int(min(max_positions, spec.max_positions) if spec.max_positions else max_positions)
        inv = inverse_frequencies(spec)
        self.rotary_dim = rotary_dim(spec)
        pairing = spec.options.get("pairing", "half")
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"rope pairing must be \"half\" or \"interleaved\", not {pairing!r}")
        self.interleaved = pairing == "interleaved"
        table = torch.empty(self.max_positions, self.rotary_dim // 2, 2, dtype=torch.float32)
        # In blocks, to bound the 64-bit scratch for long contexts.
        for p0 in range(0, self.max_positions, 1 << 15):
            p1 = min(self.max_positions, p0 + (1 << 15))
            ang = torch.arange(p0, p1, dtype=torch.float32)[:, None] * inv[None, :]
            table[p0:p1, :, 0] = ang.double().cos().float()
            table[p0:p1, :, 1] = ang.double().sin().float()
        if rt.dtype != torch.float32:
            table = table.to(rt.dtype).float()
        self.cos_sin = table.contiguous().to(rt.device)

    def rotation(self) -> Rotation:
        return Rotation(self.cos_sin, self.rotary_dim, self.interleaved)


@register_position("none")
class NoPosition(PositionEncoding):
    def __init__(self, spec, rt, max_positions):
        self.spec = spec
        self.max_positions = max_positions
