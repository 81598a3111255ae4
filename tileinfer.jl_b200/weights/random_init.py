"""Random weights from a configuration and a seed, and the model folder that holds them.

A counter-based generator: ``value = f(seed, tensor name, element index)``. A tensor's
values depend on nothing else: not on which other tensors exist, on the order in which they are
made, or on where they are made. The same function exists twice, as a CUDA kernel
(``csrc/random_init.cu``, used when the tensors are wanted on the device: an 8-billion-parameter
model is drawn in place in a fraction of a second) and here in numpy (used without a device);
both give the same bits, so ``Engine.random(config, seed)`` and
``Engine.load(write_model_folder(config, seed))`` are the same model, and anyone who restates
the function (the test-suite's plain implementation does) can regenerate what a benchmark ran.

The function: two 32-bit keys from the seed and an FNV-1a hash of the tensor's name, mixed by
lowbias32, the integer hash AntoineBut/TileInfer.jl uses for its sampling uniforms
(src/engine/sampler.jl:34-47); per element two 24-bit uniforms, then Box-Muller. Logarithm and
cosine are fixed sequences of IEEE 32-bit additions, multiplications, one division and one
square root (no library function, no fused multiply-add), which is what makes the bits portable.
Distributions come from the tensor declarations of the parts: matrices N(0, std), norm weights
1 + N(0, std), xIELU raw alphas log(e^0.8 - 1) + N(0, 0.05), beta 0.5, eps -1e-6. The reference
has no such mode; its only random model is made in Python for fixtures
(scripts/gen_apertus_fixtures.py:80-96).
"""
from __future__ import annotations

import json
import os
from typing import Dict, Sequence, Tuple

import numpy as np
import torch

from ..config.spec import TensorDecl
from ..sampling.params import mix32
from .safetensors_io import save_file

_F = np.float32
# The constants of the two series, as the 32-bit values nearest to them.
_LN_SERIES = [_F(2.0 / 9.0), _F(2.0 / 7.0), _F(2.0 / 5.0), _F(2.0 / 3.0), _F(2.0)]
_SIN_SERIES = [_F(1.0 / 362880.0), _F(-1.0 / 5040.0), _F(1.0 / 120.0), _F(-1.0 / 6.0), _F(1.0)]
_COS_SERIES = [_F(-1.0 / 3628800.0), _F(1.0 / 40320.0), _F(-1.0 / 720.0), _F(1.0 / 24.0), _F(-0.5), _F(1.0)]
_LN2, _SQRT2, _QUARTER_PI = _F(0.6931471805599453), _F(1.4142135623730951), _F(0.7853981633974483)
MAX_ELEMENTS = 1 << 32          # the element counter has 32 bits


def tensor_keys(seed: int, name: str) -> Tuple[int, int]:
    """The two 32-bit keys of tensor ``name`` under ``seed``."""
    h = 0x811C9DC5                                     # FNV-1a over the name's UTF-8 bytes
    for byte in name.encode("utf-8"):
        h = ((h ^ byte) * 0x01000193) & 0xFFFFFFFF
    k0 = mix32(mix32(seed & 0xFFFFFFFF) ^ h)
    return k0, mix32((k0 + 0x9E3779B9) & 0xFFFFFFFF)


def _mix32(x: np.ndarray) -> np.ndarray:
    x = x ^ (x >> np.uint32(16))
    x = x * np.uint32(0x7FEB352D)
    x = x ^ (x >> np.uint32(15))
    x = x * np.uint32(0x846CA68B)
    return x ^ (x >> np.uint32(16))


def _horner(coefficients, x2: np.ndarray) -> np.ndarray:
    t = np.full_like(x2, coefficients[0])
    for c in coefficients[1:]:
        t = t * x2 + c                                   # two roundings: numpy never fuses them
    return t


def standard_normal(k0: int, k1: int, first: int, count: int) -> np.ndarray:
    """z(first .. first + count) as float32, the same bits as ``csrc/random_init.cu``."""
    if first < 0 or first + count > MAX_ELEMENTS:
        raise ValueError(f"elements {first}..{first + count} are outside the 32-bit counter")
    i = (np.arange(count, dtype=np.uint64) + np.uint64(first)).astype(np.uint32)
    a = _mix32(i ^ np.uint32(k0)) >> np.uint32(8)
    b = _mix32(i ^ np.uint32(k1)) >> np.uint32(8)
    # ln u, u = (a + 1) 2^-24 in (0, 1]: n = a + 1 = m 2^e with m in (sqrt(1/2), sqrt(2)]
    bits = (a + np.uint32(1)).astype(_F).view(np.uint32)
    e = (bits >> np.uint32(23)).astype(np.int32) - 127
    m = ((bits & np.uint32(0x7FFFFF)) | np.uint32(0x3F800000)).view(_F)
    high = m > _SQRT2
    m = np.where(high, m * _F(0.5), m)
    e = e + high.astype(np.int32)
    s = (m - _F(1.0)) / (m + _F(1.0))
    ln_u = (e - 24).astype(_F) * _LN2 + s * _horner(_LN_SERIES, s * s)
    r = np.sqrt(_F(-2.0) * ln_u)
    # cos(2 pi b 2^-24), by octants of the integer b
    q = b >> np.uint32(21)
    f = (b & np.uint32(0x1FFFFF)).astype(_F) * _F(2.0 ** -21)
    g = np.where((q & np.uint32(1)) == 1, _F(1.0) - f, f)
    x = g * _QUARTER_PI
    x2 = x * x
    sine = x * _horner(_SIN_SERIES, x2)
    cosine = _horner(_COS_SERIES, x2)
    c = np.where((((q + np.uint32(1)) >> np.uint32(1)) & np.uint32(1)) == 1, sine, cosine)
    c = np.where((q >= 2) & (q <= 5), -c, c)
    return (r * c).astype(_F, copy=False)


def _moments(init) -> Tuple[float, float]:
    kind = init[0]
    if kind == "normal":
        return 0.0, float(init[1])
    if kind == "one_plus_normal":
        return 1.0, float(init[1])
    if kind == "const_plus_normal":
        return float(init[1]), float(init[2])
    raise ValueError(f"unknown init kind {kind}")


def _host_tensor(d: TensorDecl, seed: int, dtype: torch.dtype) -> torch.Tensor:
    shape = tuple(d.shape)
    count = int(np.prod(shape, dtype=np.int64)) if shape else 1
    mean, std = _moments(d.init)
    k0, k1 = tensor_keys(seed, d.name)
    out = torch.empty(count, dtype=dtype)
    block = 1 << 22                                      # bounds the 32-bit scratch of large tables
    for first in range(0, count, block):
        n = min(block, count - first)
        z = standard_normal(k0, k1, first, n)
        out[first:first + n] = torch.from_numpy(_F(mean) + z * _F(std)).to(dtype)
    return out.view(shape)


def _device_tensor(d: TensorDecl, seed: int, dtype: torch.dtype, device: str) -> torch.Tensor:
    from ..kernels import ops
    mean, std = _moments(d.init)
    k0, k1 = tensor_keys(seed, d.name)
    out = torch.empty(tuple(d.shape), dtype=dtype, device=device)
    ops.random_normal(out, k0, k1, mean, std)
    return out


def random_tensors(decls: Sequence[TensorDecl], seed: int, dtype: torch.dtype = torch.bfloat16,
                   device: str = "cpu") -> Dict[str, torch.Tensor]:
    """Tensors for ``decls``; values are computed in 32-bit and rounded once to ``dtype`` (bfloat16 or
    float32). On a CUDA ``device`` they are made there by the kernel, else here in numpy: the same bits."""
    if dtype not in (torch.bfloat16, torch.float32):
        raise ValueError(f"random weights are made in bfloat16 or float32, not {dtype}")
    on_device = torch.device(device).type == "cuda"
    out = {}
    for d in decls:
        shape = tuple(d.shape)
        count = 1
        for n in shape:
            count *= int(n)
        if count > MAX_ELEMENTS:
            raise ValueError(f"{d.name} has {count} elements; the generator's counter has 32 bits")
        if d.init[0] == "const":
            out[d.name] = torch.full(shape, float(d.init[1]), dtype=torch.float32, device=device).to(dtype)
        elif on_device:
            out[d.name] = _device_tensor(d, seed, dtype, device)
        else:
            out[d.name] = _host_tensor(d, seed, dtype)
    return out


def write_model_folder(config, seed: int, out_dir: str, dtype: torch.dtype = torch.bfloat16, device: str = None) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (a typed configuration).

    Returns ``out_dir``. The tensor list comes from the model the registry builds for the
    configuration, so the folder loads back without missing or unexpected tensors. The values are made
    on ``device`` (default: a CUDA device if there is one, which takes seconds where numpy takes minutes
    for billions of elements; the bits are the same either way).
    """
    from ..engine.model import tensor_declarations
    cfg_dict = config.to_dict()
    cfg_dict["dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32"}[dtype]
    decls = tensor_declarations(config.model_spec())
    if device is None:
        device = "cuda" if torch.cuda.is_available() else "cpu"
    tensors = {k: v.cpu() for k, v in random_tensors(decls, seed, dtype=dtype, device=device).items()}
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg_dict, f, indent=2)
        f.write("\n")
    save_file(tensors, os.path.join(out_dir, "model.safetensors"), metadata={"format": "pt", "seed": str(seed)})
    return out_dir
