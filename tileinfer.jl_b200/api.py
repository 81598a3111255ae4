"""The Python entry point, in the manner of AntoineBut/TileInfer.jl's programmatic API
(docs/src/usage.md:59-80: ``load_model(dir; T, backend, max_len)``,
``generate(model, ids; max_new_tokens, sampling, stop_ids, rng, on_token)``), widened from
one sequence to batches of requests. Token ids go in and come out; there is no tokenizer.
"""
from __future__ import annotations

import json
import os
from typing import Callable, List, Optional, Sequence, Union

from .engine import Engine
from .engine.generate import generate as _generate
from .sampling import SamplingParams

_BACKENDS = {"fast": "fast", "plain": "plain"}


def load_model(model_dir: str, dtype: str = "bfloat16", backend: str = "fast", max_context: int = 4096,
               max_tokens: Optional[int] = None, max_seqs: int = 8, **kw) -> Engine:
    """Load the model folder ``model_dir`` (config.json + safetensors) onto the GPU.

    ``dtype``: "bfloat16" or "float32" (the true 32-bit path). ``backend``: "fast" (tensor-core and
    bandwidth kernels) or "plain" (the simple reference kernels), like the reference's tile/ref.
    ``max_context`` is the longest sequence in tokens (it sizes the rotary tables); ``max_tokens`` the
    most tokens all live sequences hold together (default: ``max_seqs × max_context``)."""
    if backend not in _BACKENDS:
        raise ValueError("backend expects fast or plain")
    return Engine.load(model_dir, dtype=dtype, kernels=_BACKENDS[backend], max_context=max_context,
                       max_tokens=max_tokens or max_seqs * max_context, max_seqs=max_seqs, **kw)


def generation_defaults(model_dir: str, engine: Engine):
    """Sampling settings and stop tokens recommended by the model's generation_config.json, if it has
    one; greedy and the configuration's EOS ids otherwise (src/engine/generate.jl:83-93)."""
    stop = list(engine.spec.eos_token_ids)
    path = os.path.join(model_dir, "generation_config.json")
    if not os.path.isfile(path):
        return SamplingParams(), stop
    with open(path) as f:
        g = json.load(f)
    eos = g.get("eos_token_id")
    for e in ([] if eos is None else [eos] if isinstance(eos, int) else eos):
        if e not in stop:
            stop.append(e)
    if not g.get("do_sample", False):
        return SamplingParams(), stop
    return SamplingParams(temperature=g.get("temperature", 1.0), top_k=g.get("top_k", 0), top_p=g.get("top_p", 1.0)), stop


def generate(model: Engine, prompts: Union[Sequence[int], Sequence[Sequence[int]]], max_new_tokens: int = 256,
             sampling: SamplingParams = SamplingParams(), stop_ids: Optional[Sequence[int]] = None, seed: int = 0,
             on_token: Optional[Callable[[int, int], None]] = None):
    """Generate up to ``max_new_tokens`` tokens for one prompt (a list of ids; returns a list) or for
    several (a list of lists; returns a list of lists). Stop tokens are not returned."""
    single = len(prompts) > 0 and isinstance(prompts[0], int)
    out = _generate(model, [prompts] if single else prompts, max_new_tokens=max_new_tokens, sampling=sampling,
                    stop_ids=stop_ids, seed=seed, on_token=on_token)
    return out[0] if single else out
