"""Arrangement of a layer's parts. ``pre_norm``: x += mixer(norm1(x)); x += ffn(norm2(x)).

Each residual add is fused with the norm that follows it, so a block receives the already
normed input ``h`` and produces the next block's normed input with ``next_norm`` (the next
block's mixer norm, or the model's final norm), as AntoineBut/TileInfer.jl's step does
(src/model/decoder.jl:173-192).
"""
from __future__ import annotations

from .base import register_block


@register_block("pre_norm")
class PreNormBlock:
    def __init__(self, spec, mixer, feed_forward, mixer_norm, feed_forward_norm):
        self.spec = spec
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm

    @property
    def input_norm(self):
        return self.mixer_norm

    def forward(self, x, h, step, cache, next_norm, h_out):
        """x: residual stream (updated in place); h = input_norm(x); writes next_norm(x) to h_out."""
        delta = self.mixer.forward(h, step, cache)
        self.feed_forward_norm.add_forward(x, delta, h)
        delta = self.feed_forward.forward(h, step)
        next_norm.add_forward(x, delta, h_out)
        return h_out
