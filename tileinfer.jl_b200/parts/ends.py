"""The two ends of the model: the token embedding and the LM head.

AntoineBut/TileInfer.jl: ``x[t] = E[ids[t]]``, no scaling (src/ops/reference.jl:10); only the first
``vocab_size`` rows of the table are loaded (src/hub/loader.jl:155-156); the head is a product with
32-bit output, the value rounded to the storage type first (src/ops/tile/linear.jl:12-13, 26), and a
tied head is the embedding table itself (src/hub/loader.jl:157-163).
"""
from __future__ import annotations

from ..config.spec import ModelSpec, TensorDecl
from ..kernels import ops
from .base import Embedding, Head, register_embedding, register_head
from .linear import Linear


@register_embedding("lookup")
class TokenEmbedding(Embedding):
    def __init__(self, spec: ModelSpec, tensors, rt):
        self.table = rt.param(tensors[spec.embed_name])

    @classmethod
    def tensors(cls, spec: ModelSpec):
        return [TensorDecl(spec.embed_name, (spec.vocab_size, spec.hidden_size), ("normal", spec.init_std), allow_extra_rows=True)]

    def forward(self, token_ids, out, status):
        ops.embed(out, self.table, token_ids, status)
        return out


@register_head("linear")
class LinearHead(Head):
    def __init__(self, spec: ModelSpec, tensors, rt, embedding):
        weight = embedding.table if spec.lm_head_name is None else rt.param(tensors[spec.lm_head_name])
        self.linear = Linear(weight, rt, "lm_head")

    @classmethod
    def tensors(cls, spec: ModelSpec):
        if spec.lm_head_name is None:
            return []
        return [TensorDecl(spec.lm_head_name, (spec.vocab_size, spec.hidden_size), ("normal", spec.init_std))]

    def forward(self, h, logits):
        return self.linear.forward(h, logits, ops.EPI_F32_OUT)
