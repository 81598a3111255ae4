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

import numpy as np
import torch


def _align(n: int, a: int = 32) -> int:
    return -(-n // a) * a


@dataclass
class GroupMeta:
    slot_mapping: torch.Tensor          # [n_tokens] flat position in the pool: page * page_size + offset
    block_table: torch.Tensor           # [max_seqs, max_pages] pages of every slot
    # Decode steps only, when the planner has a split policy: how the attention kernel's B x splits work
    # slots are shared out among the sequences (see ``split_tables``).
    decode_splits: int = 0
    split_work: Optional[torch.Tensor] = None     # [B * splits, 2]
    split_seq: Optional[torch.Tensor] = None      # [B]


MAX_PARTS = 32                          # parts of one sequence in decode attention (the combine kernel's limit)


def split_tables(lengths: np.ndarray, splits: int, page_size: int):
    """Shares B x splits work slots out among B sequences of ``lengths`` keys: every sequence gets one
    part, the remaining slots go in proportion to the sequences' pages, so that a long sequence is read by
    more blocks than a short one (with equal lengths every sequence gets ``splits`` parts). A sequence's
    slots are consecutive. Returns work[slot] = (sequence << 16 | part << 8 | parts, or -1: no work; the
    sequence's length) and seq[sequence] = first slot << 8 | parts."""
    B = len(lengths)
    T = B * splits
    pages = np.maximum(-(-lengths.astype(np.int64) // page_size), 1)
    parts = 1 + ((T - B) * pages) // int(pages.sum())
    parts = np.minimum(np.minimum(parts, MAX_PARTS), pages)
    first = np.cumsum(parts) - parts
    used = int(parts.sum())
    work = np.zeros((T, 2), dtype=np.int64)
    work[:, 0] = -1
    owner = np.repeat(np.arange(B, dtype=np.int64), parts)
    work[:used, 0] = (owner << 16) | ((np.arange(used, dtype=np.int64) - first[owner]) << 8) | parts[owner]
    work[:used, 1] = lengths[owner]
    return work, (first << 8) | parts


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
        n_groups = max(1, len(cache.paged_groups))
        cap = (_align(max_step_tokens) * (3 + n_groups + 1) + 4 * _align(cache.max_seqs + 1) + 64 +
               n_groups * (_align(2 * cache.max_seqs * MAX_PARTS) + _align(cache.max_seqs)))
        self.capacity = cap
        pin = self.device.type == "cuda"
        self.staging = [torch.zeros(cap, dtype=torch.int32, pin_memory=pin) for _ in range(2)]
        self.staging_np = [t.numpy() for t in self.staging]
        self.events = [None, None]
        self.turn = 0
        self.meta = torch.zeros(cap, dtype=torch.int32, device=self.device)
        self.runtime = None
        # (batch size, paged group) -> split count of decode attention, or None: who builds the engine decides
        # (the fast kernels split, the plain ones do not).
        self.split_policy = None
        self._split_cache = {}
        self.last_upload_bytes = 0
        self._layouts = {}
        self._tables_np = [g.host_table.numpy() for g in cache.paged_groups]

    def _layout(self, n: int, B: int, nw: int):
        """Segment offsets and device views for a step of n tokens, B sequences, nw wanted rows."""
        key = (n, B, nw)
        lay = self._layouts.get(key)
        if lay is not None:
            return lay
        off = 0
        def seg(length):
            nonlocal off
            o = off
            off += _align(length)
            return o
        o = {"ids": seg(n), "pos": seg(n), "slot": seg(n)}
        o["maps"] = [seg(n) for _ in self.cache.paged_groups]
        o["seq"], o["cu"], o["kv"], o["want"] = seg(B), seg(B + 1), seg(B), seg(nw)
        o["splits"] = [0 for _ in self.cache.paged_groups]
        if n == B and self.split_policy is not None:         # a decode step
            o["splits"] = [int(self.split_policy(B, g) or 0) for g in self.cache.paged_groups]
            o["work"] = [seg(2 * B * sp) if sp > 1 else 0 for sp in o["splits"]]
            o["seqw"] = [seg(B) if sp > 1 else 0 for sp in o["splits"]]
        o["end"] = off
        m = self.meta
        views = dict(
            token_ids=m[o["ids"]:o["ids"] + n], positions=m[o["pos"]:o["pos"] + n], tok_slot=m[o["slot"]:o["slot"] + n],
            seq_slots=m[o["seq"]:o["seq"] + B], cu_seqlens=m[o["cu"]:o["cu"] + B + 1], kv_lens=m[o["kv"]:o["kv"] + B],
            want_idx=m[o["want"]:o["want"] + nw],
            groups={g.index: GroupMeta(m[o["maps"][gi]:o["maps"][gi] + n], g.device_table,
                                       **({"decode_splits": o["splits"][gi],
                                           "split_work": m[o["work"][gi]:o["work"][gi] + 2 * B * o["splits"][gi]],
                                           "split_seq": m[o["seqw"][gi]:o["seqw"][gi] + B]} if o["splits"][gi] > 1 else
                                          {"decode_splits": o["splits"][gi]}))
                    for gi, g in enumerate(self.cache.paged_groups)})
        if len(self._layouts) > 256:
            self._layouts.clear()
        lay = self._layouts[key] = (o, views)
        return lay

    def _fill_splits(self, o, st, lengths_after: np.ndarray):
        """The decode attention's work tables for sequences that hold ``lengths_after`` keys after the step;
        they change only when a sequence starts a new page, and are kept until then."""
        for gi, g in enumerate(self.cache.paged_groups):
            sp = o["splits"][gi]
            if sp <= 1:
                continue
            B = len(lengths_after)
            pages = -(-lengths_after // g.page_size)
            key = (gi, B)
            held = self._split_cache.get(key)
            if held is None or not np.array_equal(held[0], pages):
                work, seqw = split_tables(lengths_after, sp, g.page_size)
                used = int((seqw & 255).sum())
                held = (pages.copy(), work, seqw, (work[:used, 0] >> 16).copy(), used)
                self._split_cache[key] = held
            work, used = held[1], held[4]
            work[:used, 1] = lengths_after[held[3]]                        # the lengths change every step
            st[o["work"][gi]:o["work"][gi] + 2 * B * sp] = work.reshape(-1)
            st[o["seqw"][gi]:o["seqw"][gi] + B] = held[2]

    def _staging(self):
        turn = self.turn
        self.turn ^= 1
        if self.events[turn] is not None:
            self.events[turn].synchronize()          # the copy that last read this buffer has finished
        return turn, self.staging_np[turn]

    def _upload(self, turn: int, count: int, skip_ids: int = 0):
        """One copy of the first ``count`` words (without the first ``skip_ids`` when the token ids are
        written on the device)."""
        self.meta[skip_ids:count].copy_(self.staging[turn][skip_ids:count], non_blocking=True)
        self.last_upload_bytes = (count - skip_ids) * 4
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record()
            self.events[turn] = ev

    def plan(self, entries: Sequence[Tuple[int, Sequence[int]]], want: Sequence[Sequence[int]]) -> StepContext:
        """``entries``: (slot, new tokens) per sequence; ``want[i]``: offsets into entry i's tokens.
        Pages must already be reserved; lengths are those before the step."""
        cache = self.cache
        q_lens = [len(t) for _, t in entries]
        n, B = sum(q_lens), len(entries)
        nw = sum(len(w) for w in want)
        if n > self.max_step_tokens:
            raise ValueError(f"a step of {n} tokens exceeds max_step_tokens {self.max_step_tokens}")
        o, views = self._layout(n, B, nw)
        turn, st = self._staging()
        slots = [s for s, _ in entries]
        starts = [cache.length(s) for s in slots]
        row = 0
        wrow = o["want"]
        for i, (slot, toks) in enumerate(entries):
            m, start = q_lens[i], starts[i]
            pos = np.arange(start, start + m, dtype=np.int64)
            st[o["ids"] + row:o["ids"] + row + m] = toks
            st[o["pos"] + row:o["pos"] + row + m] = pos
            st[o["slot"] + row:o["slot"] + row + m] = slot
            for gi, g in enumerate(cache.paged_groups):
                P = g.page_size
                st[o["maps"][gi] + row:o["maps"][gi] + row + m] = self._tables_np[gi][slot, pos // P].astype(np.int64) * P + pos % P
            for w in want[i]:
                if not 0 <= w < m:
                    raise ValueError(f"wanted position {w} is outside the {m} tokens of entry {i}")
                st[wrow] = row + w
                wrow += 1
            st[o["cu"] + i] = row
            row += m
        st[o["cu"] + B] = row
        st[o["seq"]:o["seq"] + B] = slots
        st[o["kv"]:o["kv"] + B] = [a + b for a, b in zip(starts, q_lens)]
        if n == B and any(o["splits"]):
            self._fill_splits(o, st, np.asarray(starts, dtype=np.int64) + 1)
        self._upload(turn, o["end"])
        return StepContext(n_tokens=n, n_seqs=B, n_want=nw, host_slots=slots, host_q_lens=q_lens, host_starts=starts,
                           is_decode=all(q == 1 for q in q_lens), max_q_len=max(q_lens, default=0),
                           max_kv_len=max((a + b for a, b in zip(starts, q_lens)), default=0), runtime=self.runtime, **views)

    def plan_decode(self, slots: Sequence[int], tokens: Optional[Sequence[int]]) -> StepContext:
        """One token for each of ``slots``, the last (only) token's logits wanted. With ``tokens`` None
        the ids are left to a kernel that writes them into ``token_ids`` on the device (the sampler of
        the previous step), and only the rest is uploaded."""
        cache = self.cache
        B = len(slots)
        o, views = self._layout(B, B, B)
        turn, st = self._staging()
        slot_arr = np.asarray(slots, dtype=np.int64)
        starts = np.fromiter((cache.lengths[s] for s in slots), dtype=np.int64, count=B)
        if tokens is not None:
            st[o["ids"]:o["ids"] + B] = tokens
        st[o["pos"]:o["pos"] + B] = starts
        st[o["slot"]:o["slot"] + B] = slot_arr
        for gi, g in enumerate(cache.paged_groups):
            P = g.page_size
            st[o["maps"][gi]:o["maps"][gi] + B] = self._tables_np[gi][slot_arr, starts // P].astype(np.int64) * P + starts % P
        ar = np.arange(B + 1)
        st[o["cu"]:o["cu"] + B + 1] = ar
        st[o["seq"]:o["seq"] + B] = slot_arr
        st[o["kv"]:o["kv"] + B] = starts + 1
        st[o["want"]:o["want"] + B] = ar[:B]
        if any(o["splits"]):
            self._fill_splits(o, st, starts + 1)
        self._upload(turn, o["end"], skip_ids=_align(B) if tokens is None else 0)
        starts_l = starts.tolist()
        return StepContext(n_tokens=B, n_seqs=B, n_want=B, host_slots=list(slots), host_q_lens=[1] * B, host_starts=starts_l,
                           is_decode=True, max_q_len=1, max_kv_len=max(starts_l, default=0) + 1, runtime=self.runtime, **views)
