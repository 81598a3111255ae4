"""y = x Wᵀ for a weight kept [out, in] as the checkpoint stores it (no transposes:
AntoineBut/TileInfer.jl src/hub/loader.jl:1-6), 32-bit accumulation and one rounding
(src/ops/reference.jl:23-26). The kernel is chosen by element type, token count and sizes;
the 32-bit path always takes the CUDA-core product."""
from __future__ import annotations

import torch

from ..kernels import ops


class Linear:
    def __init__(self, weight: torch.Tensor, rt, name: str = "linear"):
        self.rt = rt
        self.weight = weight                 # [out, in], compute dtype, on the device
        self.out_features, self.in_features = weight.shape
        self.name = name

    def forward(self, x: torch.Tensor, out: torch.Tensor, epilogue: int = ops.EPI_NONE, act=(0.0, 0.0, 0.0, 0.0),
                allow_partials: bool = False):
        """Writes y to ``out`` and returns it. With ``allow_partials`` the result may instead come back
        as 32-bit partial sums ``[s, n, out]`` (a product split over k), for a consumer that adds them:
        the norm's ``add_forward``."""
        if self.rt.fast:
            from ..kernels import fast
            done = fast.linear(self, x, out, epilogue, act, allow_partials)
            if done is not None:
                return done
        ops.gemm_plain(out, x, self.weight, epilogue, act)
        return out
