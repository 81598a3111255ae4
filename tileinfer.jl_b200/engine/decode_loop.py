"""The generation loop's per-step enqueue, in one C++ call (``csrc/decode_loop.cu``).

For a batch whose next step has a captured graph, ``enqueue`` samples the rows of the last
logits on the device, starts the tokens on their way to pinned host memory, writes them into
the next step's token ids, reserves the next positions, uploads the next step's metadata and
launches its graph; ``wait`` then returns the tokens, one step behind the device, as
AntoineBut/TileInfer.jl's pipelined loop does for one sequence (src/engine/runner.jl:157-191).
"""
from __future__ import annotations

import ctypes
from typing import List, Sequence

import torch

from ..cache import OutOfPagesError
from ..kernels import host, library, ops
from ..kernels.library import KernelError


class DecodeLoop:
    def __init__(self, engine, sampler):
        self.engine, self.sampler = engine, sampler
        self._api = host.api()
        rows = sampler.seeds.shape[0]
        self._ws = ops.argmax_workspace(rows, engine.vocab_size, engine.device)
        self._h = self._api.loop_create(engine.cache.book, engine.planner.handle, rows, engine.vocab_size, sampler.seeds.data_ptr(),
                                        sampler.counters.data_ptr(), sampler.tokens.data_ptr(), self._ws[0].data_ptr(),
                                        self._ws[1].data_ptr(), self._ws[2].data_ptr())
        self._rows = 0

    def __del__(self):
        if getattr(self, "_h", None):
            self._api.loop_destroy(self._h)
            self._h = None

    def enqueue(self, logits: torch.Tensor, sampling, rows: Sequence[int], next_slots: Sequence[int]) -> torch.Tensor:
        """Sample every row of ``logits``; the rows ``rows`` (ascending) go on as the sequences ``next_slots`` in a
        step that is launched at once. Returns that step's logits buffer (None when nothing goes on). The next
        step's batch size must have a captured graph (``Engine.graph_ready``)."""
        eng = self.engine
        n = len(next_slots)
        graph = ids = out = None
        if n:
            graph = eng._graphs[n][0].raw_cuda_graph_exec()
            ids = eng.decode_token_buffer(n)
            out = eng._logits[n]
        needed, free = ctypes.c_longlong(), ctypes.c_longlong()
        rc = self._api.loop_enqueue(self._h, logits.data_ptr(), logits.stride(0), logits.shape[0], float(sampling.temperature),
                                    int(sampling.top_k), float(sampling.top_p), n, host.ints(rows), host.ints(next_slots), graph,
                                    ids.data_ptr() if n else None, library.current_stream(), ctypes.byref(needed), ctypes.byref(free))
        if rc == 4:
            raise OutOfPagesError(needed.value, free.value)
        if rc == 2:
            raise ValueError(host.last_error())
        if rc:
            raise KernelError(f"decode loop: {host.last_error()}")
        self._rows = logits.shape[0]
        library.add_launches(1 + (eng.decode_launches(n) if n else 0))
        return out

    def wait(self) -> List[int]:
        """The tokens sampled by the last ``enqueue``, in row order, once they are on the host."""
        buf = (ctypes.c_int * self._rows)()
        if self._api.loop_wait(self._h, buf, self._rows):
            raise KernelError(f"decode loop: {host.last_error()}")
        return list(buf)
