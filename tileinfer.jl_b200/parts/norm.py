"""RMSNorm: normalise in 32-bit, round, then scale by the weight in the storage type
(AntoineBut/TileInfer.jl src/ops/reference.jl:17-21); fused with the residual add that
precedes it (src/ops/tile/norm.jl:48-77). No bias, no ``1 + w``."""
from __future__ import annotations

from ..config.spec import NormSpec, TensorDecl
from ..kernels import ops
from .base import Norm, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, spec: NormSpec, tensors, rt):
        self.spec, self.rt = spec, rt
        self.weight = rt.param(tensors[spec.weight_name])
        self.eps = float(spec.eps)

    @classmethod
    def tensors(cls, spec: NormSpec):
        return [TensorDecl(spec.weight_name, (spec.size,), ("one_plus_normal", spec.options.get("init_std", 0.02)))]

    def forward(self, x, out):
        ops.rmsnorm(out, x, self.weight, self.eps)
        return out

    def add_forward(self, x, delta, out):
        """x += delta; out = norm(x). ``delta`` is [n, size] in the model's element type, or 32-bit
        partial sums [s, n, size] of a product that was split over k."""
        if delta.dim() == 3:
            ops.add_rmsnorm(x, None, self.weight, out, self.eps, partials=delta)
        else:
            ops.add_rmsnorm(x, delta, self.weight, out, self.eps)
        return out
