"""The engine: a model, its cache, and ONE step function.

``Engine.step(entries, want)`` runs the next tokens of some live sequences as one batch
from the cache and returns the logits at the wanted places. It is the only way tokens go
through the model: generation, trace replay and the benchmarks all call it. The sequences
of a step may have any lengths (whole prompts, or one token each); a step longer than
``max_step_tokens`` is cut into chunks internally, which changes no result.

AntoineBut/TileInfer.jl's counterpart runs one sequence per step
(``forward!``: src/model/decoder.jl:210-227, src/engine/runner.jl:65-102): host preparation,
one upload, the device-only step; steps of a few tokens are replayed from CUDA graphs
(src/engine/runner.jl:1-12, 86-99). The batch, the slots and the chunking are this library's
own.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..cache import Cache, DEFAULT_PAGE_SIZE
from ..config import load_config, resolve_architecture
from ..parts import Runtime
from ..weights import load_tensors, random_tensors
from .model import DecoderModel, ignorable_tensors, tensor_declarations
from ..kernels.host import nvtx_range
from .step import StepPlanner

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def require_cuda(device="cuda") -> torch.device:
    d = torch.device(device)
    if d.type != "cuda" or not torch.cuda.is_available():
        raise RuntimeError("tileinfer_b200 runs on a CUDA device only (sm_100a); there is no CPU path")
    return d


class Engine:
    def __init__(self, config, tensors: Dict[str, torch.Tensor], dtype="bfloat16", device="cuda",
                 max_tokens: int = 4096, max_seqs: int = 8, max_context: Optional[int] = None,
                 page_size: int = DEFAULT_PAGE_SIZE, max_step_tokens: int = 8192, kernels: str = "fast",
                 graphs: bool = True, model_factory=None):
        self.device = require_cuda(device)
        self.config = config
        self.dtype = _DTYPES[dtype]
        self.rt = Runtime(self.dtype, self.device, kernels)
        self.spec = config.model_spec()
        max_context = int(min(max_context or self.spec.max_positions, self.spec.max_positions))
        self.max_context = max_context
        factory = model_factory or DecoderModel
        self.model = factory(self.spec, tensors, self.rt, max_context)
        self.cache = Cache(self.model.cache_requests(), self.dtype, self.device, max_tokens=max_tokens,
                           max_seqs=max_seqs, page_size=page_size, max_seq_len=max_context,
                           share=self.model.cache_shares(), max_step_tokens=int(max_step_tokens))
        self.max_step_tokens = int(max_step_tokens)
        self.planner = StepPlanner(self.cache, self.max_step_tokens, self.device)
        self.planner.runtime = self.rt
        # A mixer may want tables of its own in the metadata of one-token steps: the first mixer of each paged
        # group is asked for its plan.
        asked = set()
        for occ, li in enumerate(self.spec.order):
            view = self.cache.layer(occ) if occ in self.cache._layer_view else None
            if view is None or not self.cache.groups[view.group_index].paged or view.group_index in asked:
                continue
            asked.add(view.group_index)
            mixer = self.model.blocks[li].mixer
            plan = mixer.decode_plan(self.cache.groups[view.group_index]) if hasattr(mixer, "decode_plan") else None
            if plan is not None:
                self.planner.attach_plan(self.cache.groups[view.group_index], plan)
        self.use_graphs = graphs
        self._graphs: Dict[int, object] = {}
        self._logits: Dict[int, torch.Tensor] = {}
        self._graph_launches: Dict[int, int] = {}
        self.vocab_size = self.spec.vocab_size

    # ---- construction
    @classmethod
    def load(cls, model_dir: str, **kw) -> "Engine":
        """From a folder with config.json and safetensors; the model class is chosen by config.json."""
        with open(os.path.join(model_dir, "config.json")) as f:
            raw = json.load(f)
        arch = resolve_architecture(raw)
        config = arch.config_class.from_dict(raw)
        spec = config.model_spec()
        tensors = load_tensors(model_dir, tensor_declarations(spec), ignorable_tensors(spec))
        return cls(config, tensors, model_factory=arch.model_factory, **kw)

    @classmethod
    def random(cls, config, seed: int = 0, **kw) -> "Engine":
        """Random weights drawn on the device (nothing is written to disk)."""
        device = require_cuda(kw.get("device", "cuda"))
        tensors = random_tensors(tensor_declarations(config.model_spec()), seed, dtype=torch.bfloat16, device=str(device))
        return cls(config, tensors, **kw)

    # ---- sequences
    def new_sequence(self) -> int:
        return self.cache.alloc_slot()

    def free_sequence(self, slot: int) -> None:
        self.cache.free_slot(slot)

    def sequence_length(self, slot: int) -> int:
        return self.cache.length(slot)

    def truncate(self, slot: int, length: int) -> None:
        """Forget the positions of a sequence after its first ``length``: the next step continues from
        there (the reference rolls a sequence back the same way, src/kv/block_manager.jl:74-81, to drop a
        token that went through the model but is not kept). Pages beyond the new length go back to the
        pool; nothing is cleared, the next tokens overwrite what was there. Layers with a per-sequence
        state, or a window whose pages were already given back, cannot roll back and raise."""
        self.cache.truncate(slot, length)

    # ---- the step
    def step(self, entries: Sequence[Tuple[int, Sequence[int]]], want: Optional[Sequence[Sequence[int]]] = None,
             out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Run ``entries`` = [(slot, next tokens)] as one batch; returns float32 logits
        ``[wanted, vocab]`` in the order of the entries and of ``want`` (offsets into each entry's
        tokens, in any order; default: each entry's last token).

        A step of one token per sequence that wants exactly those tokens' logits is replayed from a CUDA
        graph and returns the graph's own output buffer, one per batch size: the next such step of the same
        batch size overwrites it, so ``clone()`` what must outlive it (or pass ``out``, which is always
        written by launches of its own). Every other step returns a fresh tensor."""
        entries = [(int(s), list(t)) for s, t in entries]
        if want is None:
            want = [[len(t) - 1] for _, t in entries]
        want = [list(w) for w in want]
        if len(want) != len(entries):
            raise ValueError("want needs one list per entry")
        seen = set()
        for slot, toks in entries:
            if slot in seen:
                raise ValueError(f"sequence slot {slot} appears twice in one step")
            seen.add(slot)
            if not toks:
                raise ValueError("an entry of a step has no tokens")
            if min(toks) < 0 or max(toks) >= self.vocab_size:
                bad = next(t for t in toks if not 0 <= t < self.vocab_size)
                raise ValueError(f"token id {bad} is outside the vocabulary of {self.vocab_size}")
            if self.cache.length(slot) + len(toks) > self.max_context:
                raise ValueError(f"sequence would reach {self.cache.length(slot) + len(toks)} positions; "
                                 f"max context is {self.max_context}")
        # All pages first: a step that cannot be held changes nothing.
        self.cache.reserve([(s, len(t)) for s, t in entries], chunk_tokens=self.max_step_tokens)
        n_want = sum(len(w) for w in want)
        n_total = sum(len(t) for _, t in entries)
        decode = all(len(t) == 1 for _, t in entries) and all(w == [0] for w in want)
        if decode and out is None:
            return self._decode_step(entries, want)
        logits = out if out is not None else torch.empty((n_want, self.vocab_size), dtype=torch.float32, device=self.device)
        with nvtx_range("prefill" if not decode else "step"):
            return self._general_step(entries, want, logits, n_total)

    def _general_step(self, entries, want, logits, n_total):
        if n_total <= self.max_step_tokens:
            ctx = self.planner.plan(entries, want)
            self.model.forward(ctx, self.cache, logits)
            for s, t in entries:
                self.cache.advance(s, len(t))
            return logits
        for chunk_entries, chunk_want, rows in self._chunks(entries, want):
            nw = len(rows)
            self.cache.prepare([(s, len(t)) for s, t in chunk_entries])
            ctx = self.planner.plan(chunk_entries, chunk_want)
            if nw and rows == list(range(rows[0], rows[0] + nw)):
                self.model.forward(ctx, self.cache, logits[rows[0]:rows[0] + nw])
            elif nw:                                    # wanted places that are not in ascending order: through a buffer
                part = torch.empty((nw, self.vocab_size), dtype=torch.float32, device=self.device)
                self.model.forward(ctx, self.cache, part)
                logits.index_copy_(0, torch.tensor(rows, dtype=torch.long, device=self.device), part)
            else:
                self.model.forward(ctx, self.cache, None)
            for s, t in chunk_entries:
                self.cache.advance(s, len(t))
        return logits

    def _chunks(self, entries, want):
        """Cut a long step into steps of at most max_step_tokens, in token order. Yields the chunk's entries,
        their wanted offsets, and the rows of the step's result that those are."""
        cur_e, cur_w, cur_rows, room = [], [], [], self.max_step_tokens
        base = 0
        for (slot, toks), w in zip(entries, want):
            a = 0
            while a < len(toks):
                take = min(room, len(toks) - a)
                cur_e.append((slot, toks[a:a + take]))
                cur_w.append([x - a for x in w if a <= x < a + take])
                cur_rows += [base + k for k, x in enumerate(w) if a <= x < a + take]
                a += take
                room -= take
                if room == 0:
                    yield cur_e, cur_w, cur_rows
                    cur_e, cur_w, cur_rows, room = [], [], [], self.max_step_tokens
            base += len(w)
        if cur_e:
            yield cur_e, cur_w, cur_rows

    def _decode_step(self, entries, want):
        return self.decode([s for s, _ in entries], [t[0] for _, t in entries], reserved=True)

    def decode_token_buffer(self, batch: int) -> torch.Tensor:
        """Where a decode step of ``batch`` sequences reads its token ids on the device: a kernel (the
        sampler of the previous step) may write them there instead of the host uploading them."""
        return self.planner._layout(batch, batch, batch)[1]["token_ids"]

    def decode(self, slots: Sequence[int], tokens: Optional[Sequence[int]] = None, reserved: bool = False) -> torch.Tensor:
        """One token for each sequence of ``slots`` (replayed from a CUDA graph captured per batch size);
        returns float32 logits [len(slots), vocab]. With ``tokens`` None the ids are those already in
        ``decode_token_buffer(len(slots))``."""
        B = len(slots)
        if not reserved:
            for s in slots:
                if self.cache.length(s) + 1 > self.max_context:
                    raise ValueError(f"sequence would reach {self.cache.length(s) + 1} positions; max context is {self.max_context}")
            self.cache.reserve([(s, 1) for s in slots])
        logits = self._logits.get(B)
        if logits is None:
            logits = self._logits[B] = torch.empty((B, self.vocab_size), dtype=torch.float32, device=self.device)
        ctx = self.planner.plan_decode(slots, tokens)
        if not self.use_graphs:
            self.model.forward(ctx, self.cache, logits)
        else:
            held = self._graphs.get(B)
            if held is not None and held[1] != self.rt.generation:
                # A scratch buffer was reallocated since this graph was captured (a step of another size
                # needed a larger one, perhaps the eager first step of another batch size): the graph
                # points at freed memory and is captured again.
                held = None
                del self._graphs[B]
            if held is None:
                # First step of this size runs eagerly (it sizes the scratch buffers), then a capture
                # of the same launches replaces it; the capture recomputes the same values. The graph is
                # stored with the buffer generation it saw AFTER the eager step.
                self.model.forward(ctx, self.cache, logits)
                torch.cuda.current_stream().synchronize()
                from ..kernels import library
                before = library.launch_count
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    self.model.forward(ctx, self.cache, logits)
                self._graphs[B] = (graph, self.rt.generation)
                self._graph_launches[B] = library.launch_count - before
            else:
                held[0].replay()
        for s in slots:
            self.cache.advance(s, 1)
        return logits

    def graph_ready(self, batch: int) -> bool:
        """Whether a decode step of ``batch`` sequences can be replayed from its captured graph as it is."""
        held = self._graphs.get(batch) if self.use_graphs else None
        return held is not None and held[1] == self.rt.generation

    def decode_loop(self, sampler):
        """The C++ side of the generation loop for ``sampler``'s rows (``csrc/decode_loop.cu``)."""
        from .decode_loop import DecodeLoop
        return DecodeLoop(self, sampler)

    def decode_launches(self, batch: int) -> int:
        """Kernels in one captured decode step of ``batch`` sequences (0 before its first capture)."""
        return self._graph_launches.get(batch, 0)

    def check_health(self) -> None:
        """Raise if a kernel with bounded waits gave up since the last check (one small device read)."""
        from ..kernels import fast
        fast.check_status()
        code = int(self.model.status.item())
        if code:
            self.model.status.zero_()
            raise RuntimeError(f"token {code - 1} of a step had an id outside the vocabulary")

    # ---- accounting for the roofline report
    def weight_bytes(self) -> int:
        return self.model.weight_bytes()

    def kv_bytes_per_position(self) -> int:
        return self.cache.bytes_per_position()
