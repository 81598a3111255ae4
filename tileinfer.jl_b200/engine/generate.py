"""The generation loop above the step function.

Requests (lists of token ids) are run in batches, one batch after another: the prompts of
a batch, of unequal lengths, are prefilled in one step; every later step carries one
token of each sequence that is still alive. A sequence ends on a stop token (which is not
emitted) or when it has ``max_new_tokens`` tokens; it then leaves the batch and gives its
slot and pages back. No request joins a batch that has started.

Per sequence this is AntoineBut/TileInfer.jl's loop (src/engine/generate.jl:26-57): prefill,
then sample -> stop check -> append -> budget check -> one-token step. Afterwards the cache
held every token except the last sampled one, which never went through the model.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence

from ..sampling import DeviceSampler, SamplingParams, sequence_seed


@dataclass
class BatchPlan:
    """Which requests run together; pure bookkeeping, testable without a device."""
    batches: List[List[int]]


def plan_batches(prompt_lengths: Sequence[int], max_new_tokens: int, max_seqs: int, max_tokens: int,
                 page_size: int, max_context: int) -> BatchPlan:
    """Requests in order, as many per batch as slots and pages allow when every sequence grows to
    its budget (each rounded up to whole pages)."""
    batches, cur, used = [], [], 0
    for i, n in enumerate(prompt_lengths):
        if n < 1:
            raise ValueError(f"request {i} has no tokens")
        total = n + max_new_tokens
        if total > max_context:
            raise ValueError(f"prompt + max_new_tokens = {total} exceeds the max context {max_context}")
        need = -(-total // page_size) * page_size
        if need > max_tokens:
            raise ValueError(f"request {i} needs {need} cached positions; the cache holds {max_tokens}")
        if cur and (len(cur) == max_seqs or used + need > max_tokens):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += need
    if cur:
        batches.append(cur)
    return BatchPlan(batches)


def finished(token: int, generated: int, max_new_tokens: int, stop_ids) -> str:
    """What a sampled token means for its sequence: "stop" (a stop token: not emitted, sequence ends),
    "last" (emitted, budget reached) or "go"."""
    if token in stop_ids:
        return "stop"
    if generated + 1 >= max_new_tokens:
        return "last"
    return "go"


def generate(engine, prompts: Sequence[Sequence[int]], max_new_tokens: int = 256,
             sampling: SamplingParams = SamplingParams(), stop_ids: Optional[Sequence[int]] = None, seed: int = 0,
             on_token: Optional[Callable[[int, int], None]] = None) -> List[List[int]]:
    """New token ids of every request, without stop tokens. ``on_token(request, id)`` is called
    for each new token. ``stop_ids`` defaults to the configuration's EOS ids; ``[]`` disables them."""
    stop = set(engine.spec.eos_token_ids if stop_ids is None else stop_ids)
    prompts = [list(p) for p in prompts]
    results: List[List[int]] = [[] for _ in prompts]
    if max_new_tokens <= 0:
        return results
    cache = engine.cache
    plan = plan_batches([len(p) for p in prompts], max_new_tokens, cache.max_seqs, cache.max_tokens,
                        cache.page_size, engine.max_context)
    sampler = DeviceSampler(cache.max_seqs, engine.device)
    for batch in plan.batches:
        slots = {r: engine.new_sequence() for r in batch}
        try:
            sampler.reset([sequence_seed(seed, r) for r in batch])
            logits = engine.step([(slots[r], prompts[r]) for r in batch])
            decode_batch(engine, sampler, sampling, list(batch), slots, logits, results, max_new_tokens, stop, on_token)
            engine.check_health()
        finally:
            for r in list(slots):
                engine.free_sequence(slots.pop(r))
    return results


def decode_batch(engine, sampler, sampling, live, slots, logits, results, max_new_tokens, stop, on_token=None):
    """Decode one batch to its end, with the host one step behind the device.

    ``live``: the requests of the batch, in the order of the rows of ``logits`` (the logits of each
    request's last token so far); ``slots[r]``: the sequence of request ``r`` (removed, and the
    sequence freed, when the request ends); ``results[r]``: the list new tokens are appended to.
    ``generate`` calls this after the prompts' step; a caller that prefilled sequences itself with
    ``Engine.step`` may call it directly.

    Step k+1 is put on the stream BEFORE the host has seen the tokens sampled after step k: its ids are
    gathered on the device from the sampler's output, and its batch is every sequence that still has
    budget, assuming that none of them just sampled a stop token. The host then reads the tokens of
    step k while the device runs step k+1. A sequence that did sample a stop token has run through one
    step too many; its row is ignored from then on and it leaves the batch one step later, which
    changes nothing for the others. AntoineBut/TileInfer.jl pipelines its decode loop the same way
    for one sequence (src/engine/runner.jl:157-191)."""
    import torch
    loop = engine.decode_loop(sampler) if engine.use_graphs else None
    dead = set()                                       # requests known to have ended, possibly still a row of `logits`
    while live:
        rows = [row for row, r in enumerate(live) if r not in dead and len(results[r]) + 1 < max_new_tokens]
        nxt = [live[row] for row in rows]
        if loop is not None and (not nxt or engine.graph_ready(len(nxt))):
            # One call: sample, start the tokens' copy, hand them to the next step, reserve, upload, launch its graph.
            next_logits = loop.enqueue(logits, sampling, rows, [slots[r] for r in nxt])
            tokens = loop.wait()
        else:
            # The first step of a batch size (which captures its graph), or an engine without graphs: the same, step by step.
            whole = len(rows) == len(live)
            ids = engine.decode_token_buffer(len(nxt)) if nxt else None
            tokens_dev = sampler.sample(logits, sampling, also=ids if whole else None)
            host, ready = sampler.fetch_async(tokens_dev)
            next_logits = None
            if nxt:
                if not whole:
                    keep = torch.tensor(rows, dtype=torch.long, device=engine.device)
                    ids.copy_(tokens_dev[keep])
                    sampler.keep_rows(rows)
                next_logits = engine.decode([slots[r] for r in nxt], None)
            ready.synchronize()
            tokens = host.tolist()
        for row, r in enumerate(live):
            if r in dead:
                continue
            outcome = finished(tokens[row], len(results[r]), max_new_tokens, stop)
            if outcome != "stop":
                results[r].append(tokens[row])
                if on_token is not None:
                    on_token(r, tokens[row])
            if outcome != "go":
                dead.add(r)
                engine.free_sequence(slots.pop(r))
        live, logits = nxt, next_logits
