"""Sampling on the device, one row of logits per sequence.

Token ``c`` of a sequence seeded with ``s`` is a pure function of its logits, the sampling
settings and ``u = sampling_uniform(s, c)`` (AntoineBut/TileInfer.jl
src/engine/sampler.jl:1-6, 40-47); seeds and counters live on the device and the kernel
advances the counter, so a step can be replayed without host work.
"""
from __future__ import annotations

from typing import Sequence

import torch

from ..kernels import ops
from .params import SamplingParams


def _as_i32(values: Sequence[int]) -> torch.Tensor:
    return torch.tensor([v - (1 << 32) if v >= (1 << 31) else v for v in (x & 0xFFFFFFFF for x in values)],
                        dtype=torch.int32)


class DeviceSampler:
    def __init__(self, max_rows: int, device):
        self.device = device
        self.seeds = torch.zeros(max_rows, dtype=torch.int32, device=device)
        self.counters = torch.zeros(max_rows, dtype=torch.int32, device=device)
        self.tokens = torch.zeros(max_rows, dtype=torch.int32, device=device)
        pin = torch.device(device).type == "cuda"
        self._host = [torch.zeros(max_rows, dtype=torch.int32, pin_memory=pin) for _ in range(2)]
        self._turn = 0

    def reset(self, seeds: Sequence[int], counters: Sequence[int] = None) -> None:
        """Row i samples with seeds[i] from counter counters[i] (0 by default)."""
        n = len(seeds)
        self.seeds[:n].copy_(_as_i32(seeds))
        self.counters[:n].copy_(_as_i32(counters if counters is not None else [0] * n))

    def keep_rows(self, rows: Sequence[int]) -> None:
        """Compact the state to the given rows, in order (sequences that left the batch drop out)."""
        idx = torch.tensor(list(rows), dtype=torch.long, device=self.device)
        n = len(rows)
        self.seeds[:n] = self.seeds[idx]
        self.counters[:n] = self.counters[idx]

    def fetch_async(self, tokens: torch.Tensor):
        """Start copying sampled tokens to pinned host memory; returns (host tensor, event). The host reads
        them after ``event.synchronize()``, which can be one step later."""
        n = tokens.shape[0]
        host = self._host[self._turn][:n]
        self._turn ^= 1
        host.copy_(tokens, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        return host, ev

    def sample(self, logits: torch.Tensor, params: SamplingParams, also: torch.Tensor = None) -> torch.Tensor:
        """Tokens [rows] (int32, on the device) for float32 logits [rows, vocab]; ``also``: a second int32
        vector that receives the same tokens (the next step's token ids)."""
        n = logits.shape[0]
        out = self.tokens[:n]
        if params.greedy:
            ops.argmax(logits, out, also=also)
        else:
            ops.sample(logits, out, float(params.temperature), int(params.top_k), float(params.top_p),
                       self.seeds[:n], self.counters[:n], also=also)
        return out
