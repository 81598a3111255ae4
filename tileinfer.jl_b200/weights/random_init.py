"""Random weights from a configuration and a seed, and the model folder that holds them.

Every tensor draws from a generator seeded by (seed, tensor name), so its values do not
depend on which other tensors exist or on the order they are made in. Distributions come
from the tensor declarations of the parts: matrices N(0, std), norm weights 1 + N(0, std),
xIELU raw alphas log(e^0.8 - 1) + N(0, 0.05), beta 0.5, eps -1e-6. The reference has no
such mode; its only random model is made in Python for fixtures
(scripts/gen_apertus_fixtures.py:80-96).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Sequence

import torch

from ..config.spec import TensorDecl
from .safetensors_io import save_file


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF


def random_tensors(decls: Sequence[TensorDecl], seed: int, dtype: torch.dtype = torch.bfloat16,
                   device: str = "cpu") -> Dict[str, torch.Tensor]:
    """Tensors for ``decls``; values are drawn in 32-bit and rounded to ``dtype``."""
    out = {}
    for d in decls:
        g = torch.Generator(device=device)
        g.manual_seed(_tensor_seed(seed, d.name))
        kind = d.init[0]
        shape = tuple(d.shape)
        if kind == "const":
            t = torch.full(shape, float(d.init[1]), dtype=torch.float32, device=device)
        else:
            if len(shape) == 2 and shape[0] * shape[1] > (1 << 28):
                # Large tables are drawn in row blocks to bound the 32-bit scratch.
                t = torch.empty(shape, dtype=dtype, device=device)
                rows = max(1, (1 << 27) // shape[1])
                for r in range(0, shape[0], rows):
                    n = min(rows, shape[0] - r)
                    t[r:r + n] = _draw(d.init, (n, shape[1]), g, device).to(dtype)
                out[d.name] = t
                continue
            t = _draw(d.init, shape, g, device)
        out[d.name] = t.to(dtype)
    return out


def _draw(init, shape, g, device):
    kind = init[0]
    z = torch.randn(shape, generator=g, dtype=torch.float32, device=device)
    if kind == "normal":
        return z * float(init[1])
    if kind == "one_plus_normal":
        return 1.0 + z * float(init[1])
    if kind == "const_plus_normal":
        return float(init[1]) + z * float(init[2])
    raise ValueError(f"unknown init kind {kind}")


def write_model_folder(config, seed: int, out_dir: str, dtype: torch.dtype = torch.bfloat16) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (a typed configuration).

    Returns ``out_dir``. The tensor list comes from the model the registry builds for the
    configuration, so the folder loads back without missing or unexpected tensors.
    """
    from ..engine.model import tensor_declarations
    cfg_dict = config.to_dict()
    cfg_dict["dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32", torch.float16: "float16"}[dtype]
    decls = tensor_declarations(config.model_spec())
    tensors = random_tensors(decls, seed, dtype=dtype)
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg_dict, f, indent=2)
        f.write("\n")
    save_file(tensors, os.path.join(out_dir, "model.safetensors"), metadata={"format": "pt", "seed": str(seed)})
    return out_dir
