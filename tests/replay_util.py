"""Builds traces for bin/trace_run and collects the logits it writes, per (request, position)."""
from __future__ import annotations

import json
import os
import subprocess
import sys
from typing import Dict, List, Sequence, Tuple

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


class Trace:
    """Steps plus, for every wanted row of every step, which (request, position) it is."""

    def __init__(self):
        self.steps: List[dict] = []
        self.rows: Dict[int, List[Tuple[str, int]]] = {}
        self._fed: Dict[str, int] = {}

    def step(self, entries: Sequence[Tuple[str, Sequence[int], Sequence[int]]], end: Sequence[str] = ()):
        """entries: (request id, next tokens, wanted offsets)."""
        n = len(self.steps)
        rows = []
        for rid, toks, want in entries:
            base = self._fed.get(rid, 0)
            rows += [(rid, base + w) for w in want]
            self._fed[rid] = base + len(toks)
        for rid in end:
            self._fed.pop(rid, None)
        self.steps.append({"step": n, "entries": [{"id": r, "tokens": list(t), "want": list(w)} for r, t, w in entries],
                           "end": list(end)})
        if rows:
            self.rows[n] = rows
        return n

    # ---- the three ways of cutting the same requests
    def whole(self, requests: Dict[str, List[int]], tag: str = "w"):
        for rid, toks in requests.items():
            self.step([(tag + rid, toks, range(len(toks)))], end=[tag + rid])

    def tail_one_by_one(self, requests: Dict[str, List[int]], tail: int = 32, tag: str = "t"):
        for rid, toks in requests.items():
            head = max(len(toks) - tail, 1)
            self.step([(tag + rid, toks[:head], range(head))], end=[tag + rid] if head == len(toks) else [])
            for i in range(head, len(toks)):
                self.step([(tag + rid, [toks[i]], [0])], end=[tag + rid] if i == len(toks) - 1 else [])

    def batch(self, requests: Dict[str, List[int]], decode: Dict[str, int], tag: str = "b"):
        """One batch: every request's first len - decode[r] tokens together in one step, then one
        token each; a request leaves after its last token."""
        left = {r: list(t[len(t) - decode[r]:]) for r, t in requests.items()}
        first = [(tag + r, t[:len(t) - decode[r]], range(len(t) - decode[r])) for r, t in requests.items()]
        self.step(first, end=[tag + r for r in requests if not left[r]])
        live = [r for r in requests if left[r]]
        while live:
            entries = [(tag + r, [left[r].pop(0)], [0]) for r in live]
            self.step(entries, end=[tag + r for r in live if not left[r]])
            live = [r for r in live if left[r]]


def run_trace(model_dir: str, dtype: str, trace: Trace, out_dir: str, max_tokens: int, vocab: int, env=None,
              timeout: int = 600) -> Dict[Tuple[str, int], np.ndarray]:
    """Run bin/trace_run on the trace; returns logits by (request id, position)."""
    os.makedirs(out_dir, exist_ok=True)
    text = "".join(json.dumps(s) + "\n" for s in trace.steps)
    p = subprocess.run([sys.executable, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", out_dir,
                        "--max-tokens", str(max_tokens)], input=text, capture_output=True, text=True, timeout=timeout,
                       env=env)
    assert p.returncode == 0, f"trace_run failed ({p.returncode}):\n{p.stdout[-2000:]}\n{p.stderr[-4000:]}"
    done = [l for l in p.stdout.splitlines() if l.startswith("done ")]
    assert done == [f"done {s['step']}" for s in trace.steps], "trace_run must print `done <step>` after every step"
    out = {}
    for n, rows in trace.rows.items():
        a = np.fromfile(os.path.join(out_dir, f"{n}.f32"), dtype="<f4").reshape(len(rows), vocab)
        for row, key in zip(a, rows):
            out[key] = row
    return out
