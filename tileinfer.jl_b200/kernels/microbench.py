"""Micro-benchmarks of single kernels and a per-kernel timeline of a decode step.

    python -m tileinfer_b200.kernels.microbench gemv    --out 21504 --in 4096 --tokens 1 [--splits S]
    python -m tileinfer_b200.kernels.microbench gemm    --out 21504 --in 4096 --tokens 2048 [--epilogue xielu]
    python -m tileinfer_b200.kernels.microbench gemmd   --out 21504 --in 4096 --tokens 64 [--tile 160] [--splits S]
    python -m tileinfer_b200.kernels.microbench decode  --batch 8 --context 1024
    python -m tileinfer_b200.kernels.microbench prefill --tokens 2048 [--kernel mma]
    python -m tileinfer_b200.kernels.microbench inputs  --tokens 2048     (q/k norm + rotation + cache write)
    python -m tileinfer_b200.kernels.microbench addnorm --tokens 2048     (residual add + RMSNorm)
    python -m tileinfer_b200.kernels.microbench sampling --batch 8 [--out VOCAB]   (greedy and sampled choice of a token)
    python -m tileinfer_b200.kernels.microbench timeline --batch 1 --layers 8
    python -m tileinfer_b200.kernels.microbench timeline --tokens 2048 --layers 4      (a prefill step)

Products rotate over several weight matrices totalling more than the 126 MB L2, so weights
come from HBM; the kernels are replayed from a CUDA graph (as in a decode step) and timed with
CUDA events. With ``--once`` a kernel is launched a few times eagerly instead, which is the
form to put under ``ncu`` (one kernel, a few launches, a few hundred MB on the device).
``timeline`` prints start, duration and gap of every kernel of one replayed decode step of an
Apertus-8B-shaped model (CUPTI through torch.profiler), which shows the overlap that
programmatic dependent launch gives.
"""
from __future__ import annotations

import argparse
import collections
import sys

import torch

from . import fast
from .library import check, lib

APERTUS_8B_LAYER = dict(hidden=4096, heads=32, kv_heads=8, head_dim=128, intermediate=21504, vocab=131072)


def _graph_time(calls, reps=5):
    """Minimum time per call (ms) of ``calls`` (closures) captured into one graph."""
    calls[0]()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for c in calls:
            c()
    g.replay()
    torch.cuda.synchronize()
    best = None
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); g.replay(); b.record()
        torch.cuda.synchronize()
        t = a.elapsed_time(b) / len(calls)
        best = t if best is None else min(best, t)
    return best


def _weights(out, k, min_bytes=600e6, most=16):
    n = max(2, min(most, int(min_bytes // (out * k * 2)) + 1))
    return [(torch.randn(out, k, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(n)]


def bench_product(kind, out, k, n, splits, epilogue, once, tile=0, Ws=None, quiet=False):
    L = lib()
    Ws = Ws or _weights(out, k)
    x = torch.randn(n, k, device="cuda").to(torch.bfloat16)
    epi = {"none": 0, "xielu": 1, "f32": 2}[epilogue]
    if splits > 1:
        epi = 3
    y = torch.empty((splits, n, out) if epi == 3 else (n, out), device="cuda",
                    dtype=torch.float32 if epi in (2, 3) else torch.bfloat16)
    status = fast.status_word()

    def call(W):
        st = torch.cuda.current_stream().cuda_stream
        if kind == "gemv":
            check(L.ti_gemv_bf16(y.data_ptr(), out, x.data_ptr(), k, W.data_ptr(), n, out, k, splits, epi, 0.8, 1.3, 0.5, -1e-6, st), "gemv")
        elif kind == "gemmd":
            check(L.ti_gemm_tcgen05_decode(y.data_ptr(), out, x.data_ptr(), k, W.data_ptr(), n, out, k, tile, splits, epi, 0.8, 1.3, 0.5,
                                           -1e-6, status.data_ptr(), st), "gemm_tcgen05_decode")
        else:
            check(L.ti_gemm_tcgen05(y.data_ptr(), out, x.data_ptr(), k, W.data_ptr(), n, out, k, splits, epi, 0.8, 1.3, 0.5, -1e-6,
                                    status.data_ptr(), st), "gemm_tcgen05")
    if once:
        for W in Ws[:4]:
            call(W)
        torch.cuda.synchronize()
        print("launched", min(4, len(Ws)), kind, "kernels")
        return
    ms = _graph_time([(lambda W=W: call(W)) for W in Ws])
    fast.check_status()
    if quiet:
        return ms
    print(f"{kind} out={out} in={k} tokens={n} splits={splits} epilogue={epilogue}: {ms * 1e3:.1f} us, "
          f"{out * k * 2 / ms / 1e6:.0f} GB/s of weights, {2 * n * out * k / ms / 1e9:.1f} TFLOP/s")


def bench_decode_attention(batch, context, once, splits=0, heads=32, kv_heads=8, head_dim=128):
    L = lib()
    pages_per_seq = -(-context // 64)
    pages = batch * pages_per_seq
    k = torch.randn(pages, kv_heads, 64, head_dim, device="cuda").to(torch.bfloat16)
    v = torch.randn(pages, kv_heads, 64, head_dim, device="cuda").to(torch.bfloat16)
    q = torch.randn(batch, heads, head_dim, device="cuda").to(torch.bfloat16)
    table = torch.randperm(pages, device="cuda").to(torch.int32).view(batch, pages_per_seq)
    slots = torch.arange(batch, dtype=torch.int32, device="cuda")
    lens = torch.full((batch,), context, dtype=torch.int32, device="cuda")
    splits = splits or fast.decode_splits(batch, kv_heads, context)
    out = torch.empty(batch, heads, head_dim, dtype=torch.bfloat16, device="cuda")
    ws_o = torch.empty(batch, heads, splits, head_dim, device="cuda")
    ws_ml = torch.empty(batch, heads, splits, 2, device="cuda")

    def call():
        check(L.ti_attention_decode(out.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), table.data_ptr(), table.stride(0),
                                    slots.data_ptr(), lens.data_ptr(), ws_o.data_ptr(), ws_ml.data_ptr(), head_dim ** -0.5, batch,
                                    heads, kv_heads, head_dim, 64, splits, 0, torch.cuda.current_stream().cuda_stream), "decode")
    if once:
        for _ in range(3):
            call()
        torch.cuda.synchronize()
        print("launched 3 decode attention kernels")
        return
    ms = _graph_time([call] * 8)
    nbytes = 2 * batch * context * kv_heads * head_dim * 2
    print(f"decode attention batch={batch} context={context} splits={splits}: {ms * 1e3:.1f} us, {nbytes / ms / 1e6:.0f} GB/s of cache"
          + ("" if nbytes > 126e6 else " (the cache of this case fits L2)"))


def bench_prefill_attention(tokens, once, kernel="tc", heads=32, kv_heads=8, head_dim=128):
    L = lib()
    pages = -(-tokens // 64)
    k = torch.randn(pages, kv_heads, 64, head_dim, device="cuda").to(torch.bfloat16)
    v = torch.randn(pages, kv_heads, 64, head_dim, device="cuda").to(torch.bfloat16)
    q = torch.randn(tokens, heads, head_dim, device="cuda").to(torch.bfloat16)
    table = torch.arange(pages, dtype=torch.int32, device="cuda").view(1, pages)
    slots = torch.zeros(1, dtype=torch.int32, device="cuda")
    cu = torch.tensor([0, tokens], dtype=torch.int32, device="cuda")
    lens = torch.tensor([tokens], dtype=torch.int32, device="cuda")
    out = torch.empty(tokens, heads, head_dim, dtype=torch.bfloat16, device="cuda")
    tpt = 128 // (heads // kv_heads)
    status = fast.status_word()

    def call():
        st = torch.cuda.current_stream().cuda_stream
        if kernel == "tc":
            check(L.ti_attention_prefill_tc(out.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), pages, table.data_ptr(),
                                            table.stride(0), slots.data_ptr(), cu.data_ptr(), lens.data_ptr(), 1, tokens,
                                            -(-tokens // (2 * tpt)), head_dim ** -0.5, heads, kv_heads, head_dim, 64, 0,
                                            status.data_ptr(), st), "prefill_tc")
        else:
            check(L.ti_attention_prefill(out.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), table.data_ptr(), table.stride(0),
                                         slots.data_ptr(), cu.data_ptr(), lens.data_ptr(), 1, -(-tokens // tpt), head_dim ** -0.5, heads,
                                         kv_heads, head_dim, 64, 0, st), "prefill")
    if once:
        for _ in range(3):
            call()
        torch.cuda.synchronize()
        print("launched 3 prefill attention kernels")
        return
    ms = _graph_time([call] * 4)
    flops = 4 * head_dim * heads * tokens * (tokens + 1) / 2
    fast.check_status()
    print(f"prefill attention ({kernel}) tokens={tokens}: {ms * 1e3:.1f} us, {flops / ms / 1e9:.1f} TFLOP/s (causal)")


def bench_attention_inputs(tokens, once, heads=32, kv_heads=8, head_dim=128):
    """Per-head q/k norm + rotation + cache write of ``tokens`` tokens of one sequence (a prefill step's kernel)."""
    from types import SimpleNamespace

    from . import ops
    F = (heads + 2 * kv_heads) * head_dim
    pages = -(-tokens // 64)
    # Rotating inputs, as the step's activations are new every layer (they come from L2 or HBM, not from L1).
    qkvs = [torch.randn(tokens, F, device="cuda").to(torch.bfloat16) for _ in range(4)]
    q = torch.empty(tokens, heads, head_dim, dtype=torch.bfloat16, device="cuda")
    k = torch.zeros(pages, kv_heads, 64, head_dim, dtype=torch.bfloat16, device="cuda")
    v = torch.zeros_like(k)
    qn = torch.ones(head_dim, dtype=torch.bfloat16, device="cuda")
    kn = torch.ones(head_dim, dtype=torch.bfloat16, device="cuda")
    table = torch.randn(tokens, head_dim // 2, 2, device="cuda")
    rotation = SimpleNamespace(cos_sin=table, rotary_dim=head_dim, interleaved=False)
    pos = torch.arange(tokens, dtype=torch.int32, device="cuda")
    calls = [(lambda x=x: ops.attention_inputs(x, q, k, v, qn, kn, 1e-5, rotation, pos, pos, heads, kv_heads, head_dim, 64)) for x in qkvs]
    if once:
        for c in calls[:3]:
            c()
        torch.cuda.synchronize()
        print("launched 3 attention-inputs kernels")
        return
    ms = _graph_time(calls)
    nbytes = tokens * F * 2 * 2
    print(f"attention inputs tokens={tokens}: {ms * 1e3:.1f} us, {nbytes / ms / 1e6:.0f} GB/s read + written")


def bench_add_norm(tokens, once, hidden=4096):
    """Residual add + RMSNorm of ``tokens`` rows (a prefill step's kernel): reads x and delta, writes x and h."""
    from . import ops
    xs = [torch.randn(tokens, hidden, device="cuda").to(torch.bfloat16) for _ in range(4)]
    ds = [torch.randn(tokens, hidden, device="cuda").to(torch.bfloat16) for _ in range(4)]
    h = torch.empty(tokens, hidden, dtype=torch.bfloat16, device="cuda")
    w = torch.ones(hidden, dtype=torch.bfloat16, device="cuda")
    calls = [(lambda x=x, d=d: ops.add_rmsnorm(x, d, w, h, 1e-5)) for x, d in zip(xs, ds)]
    if once:
        for c in calls[:3]:
            c()
        torch.cuda.synchronize()
        print("launched 3 add + norm kernels")
        return
    ms = _graph_time(calls)
    print(f"add + norm tokens={tokens}: {ms * 1e3:.1f} us, {tokens * hidden * 2 * 4 / ms / 1e6:.0f} GB/s read + written")


def bench_sampling(batch, vocab, once):
    """The choice of a token from 32-bit logits of ``batch`` rows: greedy, and by temperature with and without
    top-k / top-p (logits of a spread that a model's have: normal, scaled by 3)."""
    from . import ops
    logits = [(3 * torch.randn(batch, vocab, device="cuda")).contiguous() for _ in range(4)]
    out = torch.empty(batch, dtype=torch.int32, device="cuda")
    seeds = torch.arange(batch, dtype=torch.int32, device="cuda")
    counters = torch.zeros(batch, dtype=torch.int32, device="cuda")
    ws = ops.argmax_workspace(batch, vocab, "cuda")
    kinds = {"greedy": lambda l: ops.argmax(l, out, ws),
             "temperature 0.8": lambda l: ops.sample(l, out, 0.8, 0, 1.0, seeds, counters),
             "temperature 1.0, top-k 40, top-p 0.9": lambda l: ops.sample(l, out, 1.0, 40, 0.9, seeds, counters)}
    for name, f in kinds.items():
        calls = [(lambda l=l: f(l)) for l in logits]
        if once:
            for c in calls[:3]:
                c()
            torch.cuda.synchronize()
            continue
        ms = _graph_time(calls)
        print(f"{name}: batch {batch}, vocabulary {vocab}: {ms * 1e3:.1f} us ({batch * vocab * 4 / ms / 1e6:.0f} GB/s of logits)")
    if once:
        print("launched 3 kernels of each kind")


def timeline(batch, layers, cached=1023, prefill_tokens=0, shape=None):
    from torch.profiler import ProfilerActivity, profile

    from ..config import ApertusConfig
    from ..engine import Engine
    s = dict(APERTUS_8B_LAYER, **(shape or {}))
    cfg = ApertusConfig.from_dict({
        "architectures": ["ApertusForCausalLM"], "num_hidden_layers": layers, "hidden_size": s["hidden"],
        "num_attention_heads": s["heads"], "num_key_value_heads": s["kv_heads"], "head_dim": s["head_dim"],
        "intermediate_size": s["intermediate"], "vocab_size": s["vocab"], "rope_theta": 12e6, "rms_norm_eps": 1e-5,
        "max_position_embeddings": 4096, "qk_norm": True, "hidden_act": "xielu"})
    eng = Engine.random(cfg, seed=0, dtype="bfloat16", max_context=4096, max_seqs=max(batch, 1),
                        max_tokens=max(batch * 1280, prefill_tokens + 64), max_step_tokens=max(prefill_tokens, 2048))
    if prefill_tokens:
        ids = torch.randint(0, s["vocab"], (prefill_tokens,)).tolist()

        def step():
            x = eng.new_sequence()
            eng.step([(x, ids)])
            eng.free_sequence(x)
    else:
        slots = [eng.new_sequence() for _ in range(batch)]
        eng.cache.reserve([(x, cached) for x in slots])
        for x in slots:
            eng.cache.advance(x, cached)
        step = lambda: eng.step([(x, [1]) for x in slots])
    for _ in range(4):
        step()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(3):
            step()
        torch.cuda.synchronize()
    evs = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA and "Mem" not in e.name]
    evs.sort(key=lambda e: e.time_range.start)
    last = evs[-(len(evs) // 3):]
    t0 = last[0].time_range.start
    what = f"prefill of {prefill_tokens} tokens" if prefill_tokens else f"replayed decode step of batch {batch}"
    print(f"{layers} layers: {len(last)} kernels in one {what}, "
          f"{last[-1].time_range.end - t0:.1f} us from first start to last end")
    prev = None
    first_layer_end = 2 + 2 * 9
    def short(name):
        return name.replace("(anonymous namespace)::", "").replace("void ", "").split("(")[0].strip()
    for e in last[:first_layer_end]:
        gap = e.time_range.start - prev if prev is not None else 0.0
        print(f"  {short(e.name)[-44:]:44s} start {e.time_range.start - t0:8.1f}  dur {e.time_range.end - e.time_range.start:6.1f}  "
              f"gap to previous end {gap:6.1f}")
        prev = e.time_range.end
    total, count = collections.Counter(), collections.Counter()
    for e in last:
        key = short(e.name).split("<")[0]
        total[key] += e.time_range.end - e.time_range.start
        count[key] += 1
    for key, v in total.most_common():
        print(f"  {key:32s} n={count[key]:4d}  total {v:8.1f} us  mean {v / count[key]:6.1f} us")


def main(argv=None):
    ap = argparse.ArgumentParser(prog="microbench")
    ap.add_argument("what", choices=["gemv", "gemm", "gemmd", "decode", "prefill", "inputs", "addnorm", "sampling", "timeline"])
    ap.add_argument("--out", type=int, default=21504)
    ap.add_argument("--in", dest="k", type=int, default=4096)
    ap.add_argument("--tokens", type=int, default=1)
    ap.add_argument("--splits", type=int, default=0, help="k slices of a product (default 1); parts of the decode attention (default: the engine's policy)")
    ap.add_argument("--tile", type=int, default=0, help="gemmd: weight rows per tile (default: the plan's)")
    ap.add_argument("--epilogue", default="none", choices=["none", "xielu", "f32"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=1024)
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--kernel", default="tc", choices=["tc", "mma"], help="prefill attention: tcgen05 or mma.sync kernel")
    ap.add_argument("--products", default="new", choices=["new", "rows128"],
                    help="timeline: the engine's choice of product kernels, or the 128-row kernel everywhere")
    ap.add_argument("--once", action="store_true", help="a few eager launches and no timing (for ncu)")
    ap.add_argument("--shape", default="", help="timeline: layer sizes other than Apertus-8B's, as hidden,heads,kv_heads,head_dim,intermediate")
    a = ap.parse_args(argv)
    if a.products == "rows128":
        fast.DECODE_PRODUCT_MAX_TOKENS = 0
    if a.what in ("gemv", "gemm", "gemmd"):
        bench_product(a.what, a.out, a.k, a.tokens, max(1, a.splits), a.epilogue, a.once, tile=a.tile)
    elif a.what == "decode":
        bench_decode_attention(a.batch, a.context, a.once, a.splits)
    elif a.what == "prefill":
        bench_prefill_attention(a.tokens if a.tokens > 1 else 2048, a.once, a.kernel)
    elif a.what == "inputs":
        bench_attention_inputs(a.tokens if a.tokens > 1 else 2048, a.once)
    elif a.what == "addnorm":
        bench_add_norm(a.tokens if a.tokens > 1 else 2048, a.once)
    elif a.what == "sampling":
        bench_sampling(a.batch, a.out if a.out != 21504 else 131072, a.once)
    else:
        shape = dict(zip(("hidden", "heads", "kv_heads", "head_dim", "intermediate"), (int(v) for v in a.shape.split(",")))) if a.shape else None
        timeline(a.batch, a.layers, prefill_tokens=a.tokens if a.tokens > 1 else 0, shape=shape)
    return 0


if __name__ == "__main__":
    sys.exit(main())
