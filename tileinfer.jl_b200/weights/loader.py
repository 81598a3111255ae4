"""Weights by tensor name.

A model declares the tensors it expects (:class:`TensorDecl`: name, shape); the loader
reads exactly those from the folder's safetensors files and raises ONE error that lists
every missing tensor, every unexpected tensor and every wrong shape. Stored dtypes are
kept: bfloat16 stays bfloat16, a tensor stored in 32-bit floating point stays 32-bit, float16
stays float16 (the reference converts the file's type straight to the run type,
src/hub/loader.jl:43-44: widening float16 to 32-bit is exact, and a bfloat16 run rounds it once),
and integer tables become int32. Parts cast what their kernels need when they are built. The reference raises on the first missing name or wrong
size (src/hub/loader.jl:36, 94-97).
"""
from __future__ import annotations

from typing import Dict, Iterable, Sequence

import torch

from ..config.spec import TensorDecl
from .safetensors_io import open_folder


class WeightsError(ValueError):
    """The checkpoint does not fit the configuration."""

    def __init__(self, model_dir, missing, unexpected, wrong_shape):
        self.missing, self.unexpected, self.wrong_shape = list(missing), list(unexpected), list(wrong_shape)
        lines = [f"checkpoint in {model_dir} does not match the configuration:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(
                f"{n} has {list(got)}, expected {list(want)} from config" for n, got, want in self.wrong_shape))
        super().__init__("\n".join(lines))


def _stored_dtype(t: torch.Tensor) -> torch.Tensor:
    if t.dtype in (torch.bfloat16, torch.float32, torch.float16):
        return t
    if t.dtype == torch.float64:
        return t.to(torch.float32)
    if t.dtype in (torch.int64, torch.int16, torch.int8, torch.uint8, torch.bool, torch.int32):
        return t.to(torch.int32)
    return t


def load_tensors(model_dir: str, decls: Sequence[TensorDecl], ignorable: Iterable[str] = (),
                 device: str = "cpu") -> Dict[str, torch.Tensor]:
    """Read the declared tensors of ``model_dir`` to ``device``.

    ``ignorable`` names may be present without being declared (a stored ``lm_head.weight``
    of a tied checkpoint, src/hub/loader.jl:157-163).
    """
    by_name, _ = open_folder(model_dir)
    declared = {d.name: d for d in decls}
    ignorable = set(ignorable)
    missing = [n for n in declared if n not in by_name]
    unexpected = sorted(n for n in by_name if n not in declared and n not in ignorable)
    wrong = []
    for name, d in declared.items():
        if name not in by_name:
            continue
        shape = by_name[name].entries[name][1]
        want = tuple(d.shape)
        ok = shape == want
        if not ok and d.allow_extra_rows and len(shape) == len(want) and shape[1:] == want[1:] and shape[0] >= want[0]:
            ok = True
        if not ok and _numel(shape) == 1 and _numel(want) == 1:
            ok = True          # a scalar may be stored as [] or [1]
        if not ok:
            wrong.append((name, shape, want))
    if missing or unexpected or wrong:
        raise WeightsError(model_dir, missing, unexpected, wrong)
    out = {}
    for name, d in declared.items():
        t = by_name[name].tensor(name)
        if d.allow_extra_rows and t.shape[0] > d.shape[0]:
            t = t[: d.shape[0]]
        t = _stored_dtype(t)
        out[name] = t.to(device) if device != "cpu" else t.clone()
    return out


def _numel(shape) -> int:
    n = 1
    for s in shape:
        n *= s
    return n
