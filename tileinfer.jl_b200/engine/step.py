"""What one step carries besides the model: which tokens, of which sequences, where.

A step is a list of ``(slot, tokens)``: the next tokens of some live sequences, of any
lengths. Tokens are flattened in that order. Everything the kernels read per step lives in
ONE device buffer of 32-bit integers that is filled by ONE copy from pinned host memory,
so that a captured decode step reads fresh values at fixed addresses
(AntoineBut/TileInfer.jl keeps its ids, positions, slots and block table in one ``meta``
vector for the same reason: src/model/decoder.jl:107-117, 137-157).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch


def _align(n: int, a: int = 32) -> int:
    return -(-n // a) * a


@dataclass
class GroupMeta:
    slot_mapping: torch.Tensor          # [n_tokens] flat position in the pool: page * page_size + offset
    block_table: torch.Tensor           # [max_seqs, max_pages] pages of every slot


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
    """Builds StepContexts into a fixed device buffer through two alternating pinned staging buffers."""

    def __init__(self, cache, max_step_tokens: int, device):
        self.cache = cache
        self.device = torch.device(device)
        self.max_step_tokens = max_step_tokens
        n_groups = max(1, len(cache.paged_groups))
        cap = _align(max_step_tokens) * (3 + n_groups + 1) + 4 * _align(cache.max_seqs + 1) + 64
        self.capacity = cap
        pin = self.device.type == "cuda"
        self.staging = [torch.zeros(cap, dtype=torch.int32, pin_memory=pin) for _ in range(2)]
        self.events = [None, None]
        self.turn = 0
        self.meta = torch.zeros(cap, dtype=torch.int32, device=self.device)
        self.runtime = None
        self.last_upload_bytes = 0

    def plan(self, entries: Sequence[Tuple[int, Sequence[int]]], want: Sequence[Sequence[int]]) -> StepContext:
        """``entries``: (slot, new tokens) per sequence; ``want[i]``: offsets into entry i's tokens.
        Pages must already be reserved; lengths are those before the step."""
        cache = self.cache
        n = sum(len(t) for _, t in entries)
        B = len(entries)
        nw = sum(len(w) for w in want)
        if n > self.max_step_tokens:
            raise ValueError(f"a step of {n} tokens exceeds max_step_tokens {self.max_step_tokens}")
        turn = self.turn
        self.turn ^= 1
        if self.events[turn] is not None:
            self.events[turn].synchronize()
        st = self.staging[turn]
        a_n, a_b = _align(n), _align(B + 1)
        off = 0
        def seg(length):
            nonlocal off
            o = off
            off += _align(length)
            return o
        o_ids, o_pos, o_slot = seg(n), seg(n), seg(n)
        o_maps = [seg(n) for _ in cache.paged_groups]
        o_seq, o_cu, o_kv, o_want = seg(B), seg(B + 1), seg(B), seg(nw)
        ids_l, pos_l, slot_l, want_l = [], [], [], []
        maps = [[] for _ in cache.paged_groups]
        cu = [0]
        starts, q_lens, slots = [], [], []
        for i, (slot, toks) in enumerate(entries):
            start = cache.length(slot)
            m = len(toks)
            ids_l.extend(toks)
            pos_l.extend(range(start, start + m))
            slot_l.extend([slot] * m)
            for gi, g in enumerate(cache.paged_groups):
                table, P = g.tables.get(slot, ()), g.page_size
                maps[gi].extend(table[p // P] * P + p % P for p in range(start, start + m))
            for w in want[i]:
                if not 0 <= w < m:
                    raise ValueError(f"wanted position {w} is outside the {m} tokens of entry {i}")
                want_l.append(cu[-1] + w)
            cu.append(cu[-1] + m)
            starts.append(start); q_lens.append(m); slots.append(slot)
        def put(o, values):
            if values:
                st[o:o + len(values)] = torch.tensor(values, dtype=torch.int32)
        put(o_ids, ids_l); put(o_pos, pos_l); put(o_slot, slot_l)
        for gi in range(len(maps)):
            put(o_maps[gi], maps[gi])
        put(o_seq, slots); put(o_cu, cu); put(o_kv, [s + q for s, q in zip(starts, q_lens)]); put(o_want, want_l)
        self.meta[:off].copy_(st[:off], non_blocking=True)
        self.last_upload_bytes = off * 4
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record()
            self.events[turn] = ev
        m = self.meta
        return StepContext(
            n_tokens=n, n_seqs=B, n_want=nw,
            token_ids=m[o_ids:o_ids + n], positions=m[o_pos:o_pos + n], tok_slot=m[o_slot:o_slot + n],
            seq_slots=m[o_seq:o_seq + B], cu_seqlens=m[o_cu:o_cu + B + 1], kv_lens=m[o_kv:o_kv + B],
            want_idx=m[o_want:o_want + nw],
            groups={g.index: GroupMeta(m[o_maps[gi]:o_maps[gi] + n], g.device_table) for gi, g in enumerate(cache.paged_groups)},
            host_slots=slots, host_q_lens=q_lens, host_starts=starts,
            is_decode=all(q == 1 for q in q_lens), max_q_len=max(q_lens, default=0),
            max_kv_len=max((s + q for s, q in zip(starts, q_lens)), default=0),
            runtime=self.runtime,
        )
