"""Grouped-query attention over the paged cache, with optional per-head q/k RMSNorm before
the rotation.

AntoineBut/TileInfer.jl: q|k|v are one fused projection with output rows in that order
(src/hub/loader.jl:75-92, 182); per-head norm over head_dim with the layer's q_norm / k_norm
weight shared by all heads, before RoPE, v untouched (src/ops/interface.jl:161-177); keys and
values go to the sequence's pages (src/ops/tile/fused.jl:61-66); causal attention over all
cached positions with the softmax scale from the record (src/model/decoder.jl:169, 176-180).
"""
from __future__ import annotations

import torch

from ..config.spec import MixerSpec, TensorDecl
from ..kernels import ops
from .base import CacheRequest, Mixer, register_mixer
from .linear import Linear


@register_mixer("attention")
class Attention(Mixer):
    def __init__(self, spec: MixerSpec, tensors, rt, position):
        self.spec, self.rt, self.position = spec, rt, position
        if spec.head_dim < 2 or spec.head_dim % 2 or spec.head_dim > ops.MAX_HEAD_DIM:
            raise ValueError(f"attention: head size {spec.head_dim} is not one the kernels take (even, at most {ops.MAX_HEAD_DIM})")
        if spec.num_kv_heads < 1 or spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"attention: {spec.num_heads} query heads do not divide into {spec.num_kv_heads} KV heads")
        n = spec.tensor_names
        p = spec.prefix
        wq, wk, wv = (rt.param(tensors[p + n[k]]) for k in ("q", "k", "v"))
        if spec.kv_source is None:
            self.qkv = Linear(torch.cat([wq, wk, wv], 0).contiguous(), rt, "qkv")
        else:
            self.qkv = Linear(wq, rt, "q")           # this layer reads another layer's keys and values
        self.o = Linear(rt.param(tensors[p + n["o"]]), rt, "o")
        # The position encoding's rotation, if it has one: the mixer knows nothing else about it.
        self.rotation = position.rotation() if position is not None else None
        self.q_norm = rt.param(tensors[p + n["q_norm"]]) if spec.qk_norm else None
        self.k_norm = rt.param(tensors[p + n["k_norm"]]) if spec.qk_norm else None

    @classmethod
    def tensors(cls, spec: MixerSpec):
        n, p = spec.tensor_names, spec.prefix
        H, D = spec.hidden_size, spec.head_dim
        std = spec.options.get("init_std", 0.02)
        out = [TensorDecl(p + n["q"], (spec.num_heads * D, H), ("normal", std)),
               TensorDecl(p + n["o"], (H, spec.num_heads * D), ("normal", std))]
        if spec.kv_source is None:
            out += [TensorDecl(p + n["k"], (spec.num_kv_heads * D, H), ("normal", std)),
                    TensorDecl(p + n["v"], (spec.num_kv_heads * D, H), ("normal", std))]
        if spec.qk_norm:
            out += [TensorDecl(p + n["q_norm"], (D,), ("one_plus_normal", std)),
                    TensorDecl(p + n["k_norm"], (D,), ("one_plus_normal", std))]
        return out

    def cache_request(self):
        if self.spec.kv_source is not None:
            return None
        return CacheRequest("paged_kv", kv_heads=self.spec.num_kv_heads, head_dim=self.spec.head_dim,
                            window=self.spec.window)

    def decode_plan(self, group):
        """The fast decode kernel reads the keys of a step's sequences in B x splits work slots; how they are
        shared out among sequences of unequal lengths is a table in the step's metadata."""
        if not (self.rt.fast and self.rt.dtype == torch.bfloat16) or self.spec.kv_source is not None:
            return None
        from ..kernels import fast
        return fast.SplitKvPlan(self.spec.num_kv_heads, group.page_size, group.num_pages * group.page_size)

    def forward(self, h, step, cache):
        s, rt = self.spec, self.rt
        n = h.shape[0]
        nq, nkv, D = s.num_heads, s.num_kv_heads, s.head_dim
        own_kv = s.kv_source is None
        qkv = rt.buffer("attention.qkv", (n, (nq + 2 * nkv) * D if own_kv else nq * D))
        # [n, features], or partial sums [s, n, features] in steps of few tokens (the inputs kernel adds them one head a warp)
        qkv = self.qkv.forward(h, qkv, allow_partials=n <= 256)
        q = rt.buffer("attention.q", (n, nq, D))
        meta = step.group(cache.group_index)
        ops.attention_inputs(qkv, q, cache.k, cache.v, self.q_norm, self.k_norm, s.qk_norm_eps,
                             self.rotation, step.positions, meta.slot_mapping, nq, nkv, D,
                             cache.page_size, write_kv=own_kv)
        attn = rt.buffer("attention.out", (n, nq * D))
        done = False
        if rt.fast:
            from ..kernels import fast
            done = fast.attention(attn, q, cache, meta, step, s)
        if not done:
            ops.attention_plain(attn, q, cache.k, cache.v, meta.block_table, step.tok_slot, step.positions,
                                s.scale, nq, nkv, D, cache.page_size, window=s.window or 0)
        proj = rt.buffer("mixer.delta", (n, s.hidden_size))
        return self.o.forward(attn, proj, allow_partials=True)
