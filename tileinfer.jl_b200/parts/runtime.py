"""What every part needs from its surroundings: element type, device, scratch buffers.

Scratch buffers are named and grow to the largest request seen; two parts that never run
at the same time may share a name. After a first step of a given size nothing is
allocated any more, which is what lets decode steps be captured in CUDA graphs.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch


class Runtime:
    def __init__(self, dtype: torch.dtype, device: str = "cuda", kernels: str = "fast"):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"the model runs in float32 or bfloat16, not {dtype}")
        if kernels not in ("fast", "plain"):
            raise ValueError("kernels must be \"fast\" or \"plain\"")
        self.dtype = dtype
        self.device = torch.device(device)
        # "plain": only the simple CUDA-core kernels, also in bfloat16. The 32-bit path always uses them.
        self.kernels = "plain" if dtype == torch.float32 else kernels
        self._buffers: Dict[str, torch.Tensor] = {}
        self._views: Dict[tuple, torch.Tensor] = {}     # (name, shape, dtype) -> the view handed out last time
        # Counts (re)allocations of scratch buffers: a captured CUDA graph holds the addresses of the
        # buffers it was captured with and must be dropped when this number changes.
        self.generation = 0

    @property
    def fast(self) -> bool:
        return self.kernels == "fast"

    def buffer(self, name: str, shape: Tuple[int, ...], dtype: torch.dtype = None) -> torch.Tensor:
        dtype = dtype or self.dtype
        key = (name, shape, dtype)
        view = self._views.get(key)
        if view is not None:                        # the same request as before: the same view (making one costs microseconds)
            return view
        count = 1
        for s in shape:
            count *= int(s)
        buf = self._buffers.get(name)
        if buf is None or buf.dtype != dtype or buf.numel() < count:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError(f"scratch buffer {name} would be allocated during graph capture")
            buf = torch.empty(max(count, 1), dtype=dtype, device=self.device)
            self._buffers[name] = buf
            self.generation += 1
            for k in [k for k in self._views if k[0] == name]:
                del self._views[k]
        if len(self._views) > 4096:
            self._views.clear()
        view = self._views[key] = buf[:count].view(*shape)
        return view

    def param(self, t: torch.Tensor, keep_dtype: bool = False) -> torch.Tensor:
        """A checkpoint tensor on the device, in the element type the kernels compute with."""
        t = t.to(self.device)
        if not keep_dtype and t.is_floating_point():
            t = t.to(self.dtype)
        return t.contiguous()
