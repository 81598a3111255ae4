"""The non-gated feed-forward of Apertus: up_proj -> xIELU -> down_proj, no biases.

AntoineBut/TileInfer.jl: xIELU(x) = x > 0 ? ap·x·x + b·x : (expm1(min(x, e)) − x)·an + b·x
with a rounding after every operation (src/ops/reference.jl:49-56); the four scalars come
from the checkpoint's raw parameters: b = T(beta), ap = T(softplus(alpha_p)),
an = T(b + T(softplus(alpha_n))), e = T(eps), softplus on the 32-bit value
(src/hub/loader.jl:193-202). The activation is the up projection's epilogue.
"""
from __future__ import annotations

import torch

from ..config.spec import FeedForwardSpec, TensorDecl
from ..kernels import ops
from .base import FeedForward, register_feed_forward
from .linear import Linear


def xielu_scalars(alpha_p_raw, alpha_n_raw, beta_raw, eps_raw, dtype):
    r = (lambda t: t) if dtype == torch.float32 else (lambda t: t.to(dtype).float())
    f = lambda t: t.detach().float().cpu().reshape(())
    softplus = lambda t: torch.log1p(torch.exp(t))
    beta = r(f(beta_raw))
    alpha_p = r(softplus(f(alpha_p_raw)))
    alpha_n = r(beta + r(softplus(f(alpha_n_raw))))
    eps = r(f(eps_raw))
    return float(alpha_p), float(alpha_n), float(beta), float(eps)


@register_feed_forward("xielu_mlp")
class XieluMLP(FeedForward):
    def __init__(self, spec: FeedForwardSpec, tensors, rt):
        self.spec, self.rt = spec, rt
        n, p = spec.tensor_names, spec.prefix
        self.up = Linear(rt.param(tensors[p + n["up"]]), rt, "up")
        self.down = Linear(rt.param(tensors[p + n["down"]]), rt, "down")
        self.act = xielu_scalars(tensors[p + n["alpha_p"]], tensors[p + n["alpha_n"]], tensors[p + n["beta"]],
                                 tensors[p + n["eps"]], rt.dtype)

    @classmethod
    def tensors(cls, spec: FeedForwardSpec):
        n, p, o = spec.tensor_names, spec.prefix, spec.options
        std = o.get("init_std", 0.02)
        raw, raw_std = o.get("init_alpha_raw", 0.2), o.get("init_alpha_std", 0.05)
        return [
            TensorDecl(p + n["up"], (spec.intermediate_size, spec.hidden_size), ("normal", std)),
            TensorDecl(p + n["down"], (spec.hidden_size, spec.intermediate_size), ("normal", std)),
            TensorDecl(p + n["alpha_p"], (1,), ("const_plus_normal", raw, raw_std), keep_dtype=True),
            TensorDecl(p + n["alpha_n"], (1,), ("const_plus_normal", raw, raw_std), keep_dtype=True),
            TensorDecl(p + n["beta"], (), ("const", o.get("init_beta", 0.5)), keep_dtype=True),
            TensorDecl(p + n["eps"], (), ("const", o.get("init_eps", -1e-6)), keep_dtype=True),
        ]

    def forward(self, h, step):
        n = h.shape[0]
        act = self.rt.buffer("feed_forward.act", (n, self.spec.intermediate_size))
        self.up.forward(h, act, ops.EPI_XIELU, self.act)
        out = self.rt.buffer("feed_forward.delta", (n, self.spec.hidden_size))
        return self.down.forward(act, out, allow_partials=True)
