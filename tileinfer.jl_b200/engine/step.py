"""What one step carries besides the model: which tokens, of which sequences, where.

A step is a list of ``(slot, tokens)``: the next tokens of some live sequences, of any
lengths. Tokens are flattened in that order. Everything the kernels read per step lives in
ONE device buffer of 32-bit integers that is filled by ONE copy from pinned host memory,
so that a captured decode step reads fresh values at fixed addresses
(AntoineBut/TileInfer.jl keeps its ids, positions, slots and block table in one ``meta``
vector for the same reason: src/model/decoder.jl:107-117, 137-157).

The buffer is laid out and filled by the C++ host runtime (``csrc/host/step_planner.cpp``);
this module hands it the step and wraps the buffer's segments as tensors. A mixer whose
decode kernels want tables of their own in that buffer (how decode attention shares its
work slots among sequences of unequal lengths, for one) gives the planner a *plan*
(``Mixer.decode_plan``): the planner reserves the words the plan asks for and lets it fill
them every step, and knows nothing else about it.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch

from ..kernels import host


@dataclass
class GroupMeta:
    slot_mapping: torch.Tensor          # [n_tokens] flat position in the pool: page * page_size + offset
    block_table: torch.Tensor           # [max_seqs, max_pages] pages of every slot
    # One-token steps only: the plan of the group's mixer (what ``Mixer.decode_plan`` returned) and the words
    # it filled for this step, or None.
    plan: Optional[object] = None
    plan_table: Optional[torch.Tensor] = None


@dataclass
class StepContext:
    n_tokens: int
    n_seqs: int
    n_want: int
    token_ids: torch.Tensor             # [n_tokens]
    positions: torch.Tensor             # [n_tokens] position of each token in its sequence
    tok_slot: torch.Tensor              # [n_tokens] cache slot of each token's sequence
    seq_slots: torch.Tensor             # [n_seqs]
    cu_seqlens: torch.Tensor            # [n_seqs + 1] token ranges of the sequences
    kv_lens: torch.Tensor               # [n_seqs] cached length of each sequence after this step
    want_idx: torch.Tensor              # [n_want] flat token indices whose logits are wanted
    groups: dict                        # cache group index -> GroupMeta, for the paged groups
    # Host copies, for parts that choose kernels or walk sequences themselves.
    host_slots: List[int] = field(default_factory=list)
    host_q_lens: List[int] = field(default_factory=list)
    host_starts: List[int] = field(default_factory=list)
    is_decode: bool = False
    max_q_len: int = 0
    max_kv_len: int = 0
    runtime: object = None              # scratch buffers for kernels that need a workspace

    def group(self, index: int) -> GroupMeta:
        return self.groups[index]


class StepPlanner:
    """Builds StepContexts into a fixed device buffer through two alternating pinned staging buffers.

    The layout of the buffer depends only on (tokens, sequences, wanted rows), so a decode step of a
    given batch size always finds its values at the same addresses (what a captured graph needs), and
    the tensor views of a layout are made once and reused."""

    def __init__(self, cache, max_step_tokens: int, device):
        self.cache = cache
        self.device = torch.device(device)
        self.max_step_tokens = max_step_tokens
        self._api = host.api()
        self._on_device = self.device.type == "cuda"
        self._h = self._api.planner_create(cache.book, max_step_tokens, int(self._on_device))
        self._plans = {}                # paged group's place among the paged groups -> the mixer's plan
        self.meta = None
        self.runtime = None
        self._layouts = {}

    def __del__(self):
        if getattr(self, "_h", None):
            self._api.planner_destroy(self._h)
            self._h = None

    @property
    def handle(self):
        return self._h

    def attach_plan(self, group, plan) -> None:
        """``plan``: what the mixer of paged ``group`` returned from ``decode_plan``; its ``native`` field is a C++
        GroupPlan, which the planner owns from now on. Plans are attached before the first step."""
        if self.meta is not None:
            raise RuntimeError("plans are attached before the planner's first step")
        self._api.planner_attach_plan(self._h, group.book_index, plan.native)
        self._plans[group.book_index] = plan

    def _ensure_meta(self):
        if self.meta is None:
            self.capacity = self._api.planner_capacity(self._h)
            self.meta = torch.zeros(self.capacity, dtype=torch.int32, device=self.device)
            self._api.planner_set_meta(self._h, self.meta.data_ptr())

    @property
    def last_upload_bytes(self) -> int:
        return int(self._api.planner_last_upload_bytes(self._h))

    def _stream(self):
        if not self._on_device:
            return None
        from ..kernels import library
        return library.current_stream()

    def _layout(self, n: int, B: int, nw: int):
        """Segment offsets and device views for a step of n tokens, B sequences, nw wanted rows."""
        key = (n, B, nw)
        lay = self._layouts.get(key)
        if lay is not None:
            return lay
        self._ensure_meta()
        groups = self.cache.paged_groups
        raw = (ctypes.c_int * (8 + 3 * len(groups)))()
        self._api.planner_layout(self._h, n, B, nw, raw)
        o = dict(zip(("ids", "pos", "slot", "seq", "cu", "kv", "want", "end"), raw[:8]))
        o["maps"] = [raw[8 + 3 * gi] for gi in range(len(groups))]
        o["plan"] = [raw[9 + 3 * gi] for gi in range(len(groups))]
        o["plan_words"] = [raw[10 + 3 * gi] for gi in range(len(groups))]
        m = self.meta
        metas = {}
        for gi, g in enumerate(groups):
            words = o["plan_words"][gi]
            metas[g.index] = GroupMeta(m[o["maps"][gi]:o["maps"][gi] + n], g.device_table, self._plans.get(g.book_index),
                                       m[o["plan"][gi]:o["plan"][gi] + words] if words else None)
        views = dict(
            token_ids=m[o["ids"]:o["ids"] + n], positions=m[o["pos"]:o["pos"] + n], tok_slot=m[o["slot"]:o["slot"] + n],
            seq_slots=m[o["seq"]:o["seq"] + B], cu_seqlens=m[o["cu"]:o["cu"] + B + 1], kv_lens=m[o["kv"]:o["kv"] + B],
            want_idx=m[o["want"]:o["want"] + nw], groups=metas)
        if len(self._layouts) > 256:
            self._layouts.clear()
        lay = self._layouts[key] = (o, views)
        return lay

    def plan(self, entries: Sequence[Tuple[int, Sequence[int]]], want: Sequence[Sequence[int]]) -> StepContext:
        """``entries``: (slot, new tokens) per sequence; ``want[i]``: offsets into entry i's tokens.
        Pages must already be reserved; lengths are those before the step."""
        q_lens = [len(t) for _, t in entries]
        n, B = sum(q_lens), len(entries)
        nw = sum(len(w) for w in want)
        if n > self.max_step_tokens:
            raise ValueError(f"a step of {n} tokens exceeds max_step_tokens {self.max_step_tokens}")
        _, views = self._layout(n, B, nw)
        slots = [s for s, _ in entries]
        starts = [self.cache.length(s) for s in slots]
        rc = self._api.planner_plan(self._h, B, host.ints(slots), host.ints(q_lens), host.ints(t for _, toks in entries for t in toks),
                                    host.ints(len(w) for w in want), host.ints(x for w in want for x in w), self._stream())
        if rc:
            raise ValueError(host.last_error())
        return StepContext(n_tokens=n, n_seqs=B, n_want=nw, host_slots=slots, host_q_lens=q_lens, host_starts=starts,
                           is_decode=all(q == 1 for q in q_lens), max_q_len=max(q_lens, default=0),
                           max_kv_len=max((a + b for a, b in zip(starts, q_lens)), default=0), runtime=self.runtime, **views)

    def plan_decode(self, slots: Sequence[int], tokens: Optional[Sequence[int]]) -> StepContext:
        """One token for each of ``slots``, the last (only) token's logits wanted. With ``tokens`` None
        the ids are left to a kernel that writes them into ``token_ids`` on the device (the sampler of
        the previous step), and only the rest is uploaded."""
        B = len(slots)
        _, views = self._layout(B, B, B)
        starts = (ctypes.c_longlong * B)()
        rc = self._api.planner_plan_decode(self._h, B, host.ints(slots), host.ints(tokens) if tokens is not None else None,
                                           self._stream(), starts)
        if rc:
            raise ValueError(host.last_error())
        starts_l = list(starts)
        return StepContext(n_tokens=B, n_seqs=B, n_want=B, host_slots=list(slots), host_q_lens=[1] * B, host_starts=starts_l,
                           is_decode=True, max_q_len=1, max_kv_len=max(starts_l, default=0) + 1, runtime=self.runtime, **views)
