#!/usr/bin/env python3
"""Benchmark of the serving step on ONE GPU: decode tokens per second of an Apertus-8B-shaped
model with random weights (bfloat16), plus prefill throughput and roofline fractions.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--dtype bfloat16|float32] [--impl reference]
    python bench.py --preset 8b-long | 70b        (the other two sizes the reference names; a line each)

Prints one JSON line. A "step" is one decode step of the whole batch (default batch 8, every
sequence after 1,023 cached positions, context 4,096). ``value`` is decoded tokens per second
timed on the device with CUDA events around K graph-replayed steps; ``e2e`` is the same
through the Python entry point (``tileinfer_b200.generate``), host token ids in and out.
``prefill`` is one 2,048-token prompt; ``roofline`` relates the decode step's bytes (every weight
the step reads once + the live cache) to the HBM peak. ``points`` holds, flat, decode at batch 1 and
64 (``decode_bN`` tokens per second, ``decode_bN_ms`` per step, ``decode_bN_frac`` of the HBM peak,
``e2e_bN`` through the entry point) and the true 32-bit path at batch 8 (``decode_fp32_b8*``).
``--dtype float32`` makes the 32-bit path the headline instead.

Timing: W >= 3 warm-up steps; every step reads all weights (16 GB), far more than the 126 MB
L2, so no flush is needed between steps; SM clocks and throttle reasons are sampled with
nvidia-smi during the timed region.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# The configuration the reference quotes its headline numbers on: Apertus-8B sizes.
APERTUS_8B = {
    "architectures": ["ApertusForCausalLM"], "model_type": "apertus",
    "num_hidden_layers": 32, "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 128, "intermediate_size": 21504, "vocab_size": 131072, "rope_theta": 12000000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "original_max_position_embeddings": 8192,
                     "low_freq_factor": 1.0, "high_freq_factor": 4.0},
    "rms_norm_eps": 1e-5, "qk_norm": True, "tie_word_embeddings": False, "hidden_act": "xielu",
    "max_position_embeddings": 4096, "attention_bias": False, "mlp_bias": False,
}
# Apertus-70B sizes: 141 GB of weights on one GPU.
APERTUS_70B = dict(APERTUS_8B, num_hidden_layers=80, hidden_size=8192, num_attention_heads=64, intermediate_size=43008,
                   max_position_embeddings=2048)
CONTEXT = 4096
CACHED = 1023           # positions every sequence holds before the timed decode steps
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# The 32-bit path runs on the FMA pipe: 148 SMs x 128 lanes x 2 flops x 1.965 GHz (nominal; nothing measures it here).
FP32_TFLOPS = 148 * 128 * 2 * 1.965e9 / 1e12


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                p = json.load(f)
            return {k: float(p.get(k, FALLBACK_PEAKS[k])) for k in FALLBACK_PEAKS}, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
        sm = sorted(int(s[0]) for s in self.samples if s and s[0].isdigit())
        mx = [int(s[1]) for s in self.samples if len(s) > 1 and s[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for s in self.samples if len(s) >= 6 for n, v in zip(names, s[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


def fill_cache(engine, batch, cached, seed=0):
    """``batch`` live sequences with ``cached`` positions each. The cache's contents do not change the
    work of a decode step, so they are drawn at random instead of being prefilled."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(seed)
    for grp in engine.cache.paged_groups:
        for pool in (grp.k, grp.v):
            for l in range(pool.shape[0]):
                pool[l].copy_(torch.randn(pool[l].shape, generator=g, device="cuda", dtype=torch.float32).to(pool.dtype))
    slots = [engine.new_sequence() for _ in range(batch)]
    engine.cache.reserve([(s, cached) for s in slots])
    for s in slots:
        engine.cache.advance(s, cached)
    return slots


def release(engine, slots):
    for s in slots:
        engine.free_sequence(s)


def time_decode(engine, batch, steps, warmup, vocab, count_launches=False, cached=None):
    """Device time of ``steps`` decode steps of ``batch`` sequences through the library's own decode
    loop (greedy sampling on the device, the host one step behind): CUDA events are recorded when the
    tokens of step W and of step W + K reach the host, which brackets exactly K steps on the stream."""
    import torch
    from tileinfer_b200.engine.generate import decode_batch
    from tileinfer_b200.sampling import DeviceSampler, SamplingParams
    warmup = max(warmup, 3)
    cached = CACHED if cached is None else cached
    slots_list = fill_cache(engine, batch, cached - 1)
    sampler = DeviceSampler(batch, engine.device)
    gen = torch.Generator().manual_seed(1)
    tokens = torch.randint(0, vocab, (batch,), generator=gen).tolist()
    logits = engine.decode(slots_list, tokens)                       # position cached - 1: now `cached` positions are held
    slots = dict(enumerate(slots_list))
    results = [[] for _ in range(batch)]
    marks = {}

    def on_token(request, token):
        if request == 0 and len(results[0]) in (warmup, warmup + steps):
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            marks[len(results[0])] = ev
    decode_batch(engine, sampler, SamplingParams(), list(range(batch)), slots, logits, results, warmup + steps + 2, set(), on_token)
    torch.cuda.synchronize()
    ms = marks[warmup].elapsed_time(marks[warmup + steps])
    launches = engine.decode_launches(batch) + 1 if count_launches else 0     # the captured step + sampling (which hands the ids over)
    kv_positions = batch * (cached + warmup + 1 + steps / 2)
    assert not slots                                                  # the loop freed every sequence
    return ms / steps, kv_positions, launches


def time_prefill(engine, tokens, vocab, reps=3):
    import torch
    gen = torch.Generator().manual_seed(2)
    best = None
    for r in range(reps + 1):
        ids = torch.randint(0, vocab, (tokens,), generator=gen).tolist()
        s = engine.new_sequence()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        engine.step([(s, ids)])
        b.record()
        torch.cuda.synchronize()
        engine.free_sequence(s)
        if r > 0:                                       # the first run sizes the scratch buffers
            best = a.elapsed_time(b) if best is None else min(best, a.elapsed_time(b))
    return best


def time_e2e(engine, batch, steps, vocab, sample_clocks=False):
    """Decode rate through the public entry point: ``generate`` with host token ids in and out. The clock
    runs from the second generated token of the batch to the last (the reference's stats line does the
    same, src/cli.jl:177-187). Besides the mean, the arrival times give the median step and the mean of
    the first 16 steps: right after the prompts' step, which runs into the power cap, the SM clock comes
    back up over some tens of steps, and a gap between mean and median that closes with more steps is that
    ramp, not host time (host time would show in the median as well)."""
    import torch
    import tileinfer_b200 as ti
    gen = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, vocab, (CACHED,), generator=gen).tolist() for _ in range(batch)]
    stamps = []

    def on_token(request, token):
        if request == 0:
            stamps.append(time.perf_counter())         # the token is on the host: no synchronisation needed
    clocks = ClockSampler() if sample_clocks else None
    if clocks:
        clocks.start()
    ti.generate(engine, prompts, max_new_tokens=steps + 2, stop_ids=[], on_token=on_token)
    torch.cuda.synchronize()
    clock_info = clocks.stop() if clocks else None
    gaps = sorted(b - a for a, b in zip(stamps[1:], stamps[2:]))
    first = [b - a for a, b in zip(stamps[1:17], stamps[2:18])]
    n_steps = len(stamps) - 2
    span = stamps[-1] - stamps[1]
    out = {"value": round(batch * n_steps / span, 1), "unit": "tok/s", "steps": n_steps, "ms_mean": round(1e3 * span / n_steps, 4),
           "ms_median": round(1e3 * gaps[len(gaps) // 2], 4), "ms_first16": round(1e3 * sum(first) / max(len(first), 1), 4)}
    if clock_info:
        out["sm_mhz"] = clock_info["sm_mhz"]
    return out


def decode_from(engine, slots_list, logits, steps, warmup):
    """ms per step of ``steps`` decode steps after ``warmup`` of them, through the library's decode loop,
    for sequences that were prefilled (``logits`` are those of the prompts' last tokens)."""
    import torch
    from tileinfer_b200.engine.generate import decode_batch
    from tileinfer_b200.sampling import DeviceSampler, SamplingParams
    batch = len(slots_list)
    sampler = DeviceSampler(batch, engine.device)
    slots = dict(enumerate(slots_list))
    results = [[] for _ in range(batch)]
    marks = {}

    def on_token(request, token):
        if request == 0 and len(results[0]) in (warmup, warmup + steps):
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            marks[len(results[0])] = ev
    decode_batch(engine, sampler, SamplingParams(), list(range(batch)), slots, logits, results, warmup + steps + 2, set(), on_token)
    torch.cuda.synchronize()
    return marks[warmup].elapsed_time(marks[warmup + steps]) / steps


def timed_step(engine, entries):
    import torch
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    logits = engine.step(entries)
    b.record()
    torch.cuda.synchronize()
    return logits, a.elapsed_time(b)


def run_long_context(args, pk, pk_source):
    """Apertus-8B sizes with 65,536 positions: 8 prompts of unequal lengths drawn uniformly from
    [512, 32,768], prefilled together (in chunks of 8,192 tokens), then 256 decode steps."""
    import torch
    from tileinfer_b200.config import ApertusConfig
    from tileinfer_b200.engine import Engine
    cfg_dict = dict(APERTUS_8B, max_position_embeddings=65536)
    if args.layers:
        cfg_dict["num_hidden_layers"] = args.layers
    cfg = ApertusConfig.from_dict(cfg_dict)
    gen = torch.Generator().manual_seed(4)
    lengths = torch.randint(512, 32769, (8,), generator=gen).tolist()
    steps, warmup = 256 - 8, 6
    room = sum(-(-(n + 256 + 2) // 64) * 64 for n in lengths)
    engine = Engine.random(cfg, seed=0, dtype="bfloat16", max_context=65536, max_seqs=8, max_tokens=room, max_step_tokens=8192)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist() for n in lengths]
    warm = engine.new_sequence()                         # sizes the scratch buffers and loads the kernels
    engine.step([(warm, prompts[0][:8192] * 2)])
    engine.free_sequence(warm)
    slots = [engine.new_sequence() for _ in prompts]
    clocks = ClockSampler()
    clocks.start()
    logits, prefill_ms = timed_step(engine, list(zip(slots, prompts)))
    ms_step = decode_from(engine, slots, logits, steps, warmup)
    clock_info = clocks.stop()
    engine.check_health()
    weight_bytes = engine.weight_bytes()
    kv_bytes = (sum(lengths) + 8 * (warmup + 1 + steps / 2)) * engine.kv_bytes_per_position()
    achieved = (weight_bytes + kv_bytes) / (ms_step * 1e-3) / 1e9
    H, I, D, nq, nkv = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
    flops = cfg.num_hidden_layers * sum(2 * n * (H * (nq + 2 * nkv) * D + nq * D * H + 2 * H * I) + 4 * D * nq * n * (n + 1) // 2
                                        for n in lengths)
    print(json.dumps({
        "metric": "decode tok/s (Apertus-8B bf16, 8 sequences of 512 to 32,768 positions)", "value": round(8000.0 / ms_step, 1),
        "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": round(ms_step, 4), "dtype": "bf16",
        "data": "synthetic: random weights, uniform random token ids",
        "config": {"model": "Apertus-8B shapes", "layers": cfg.num_hidden_layers, "layers_full": 32, "global_batch": 8,
                   "prompt_tokens": sum(lengths), "longest": max(lengths), "shortest": min(lengths), "max_positions": 65536,
                   "prefill_chunk": 8192, "peaks": pk_source},
        "clocks": clock_info,
        "prefill": {"value": round(sum(lengths) * 1000.0 / prefill_ms, 1), "tokens": sum(lengths), "ms": round(prefill_ms, 2),
                    "frac": round(flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)}}))
    return 0


def run_70b(args, pk, pk_source):
    """Apertus-70B sizes (141 GB of weights): a 1,024-token prompt each, then decode at batch 1 and 8."""
    import torch
    from tileinfer_b200.config import ApertusConfig
    from tileinfer_b200.engine import Engine
    cfg_dict = dict(APERTUS_70B)
    if args.layers:
        cfg_dict["num_hidden_layers"] = args.layers
    cfg = ApertusConfig.from_dict(cfg_dict)
    engine = Engine.random(cfg, seed=0, dtype="bfloat16", max_context=2048, max_seqs=8, max_tokens=8 * 1344, max_step_tokens=8192)
    weight_bytes = engine.weight_bytes()
    gen = torch.Generator().manual_seed(5)
    steps, warmup = max(8, args.steps), max(args.warmup, 3)
    out = {}
    clocks = ClockSampler()
    clocks.start()
    for batch in (1, 8):
        prompts = [torch.randint(0, cfg.vocab_size, (1024,), generator=gen).tolist() for _ in range(batch)]
        slots = [engine.new_sequence() for _ in prompts]
        logits, prefill_ms = timed_step(engine, list(zip(slots, prompts)))
        if batch == 1:                                   # again, with the scratch buffers sized
            engine.free_sequence(slots[0])
            slots = [engine.new_sequence()]
            logits, prefill_ms = timed_step(engine, list(zip(slots, prompts)))
            out["prefill_1024"] = prefill_ms
        ms = decode_from(engine, slots, logits, steps, warmup)
        kv = batch * (1024 + warmup + 1 + steps / 2) * engine.kv_bytes_per_position()
        out[batch] = (ms, (weight_bytes + kv) / (ms * 1e-3) / 1e9)
    clock_info = clocks.stop()
    engine.check_health()
    H, I, D, nq, nkv = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
    flops = cfg.num_hidden_layers * (2 * 1024 * (H * (nq + 2 * nkv) * D + nq * D * H + 2 * H * I) + 4 * D * nq * 1024 * 1025 // 2)
    print(json.dumps({
        "metric": "decode tok/s (Apertus-70B bf16, batch 8, 1,024 cached positions)", "value": round(8000.0 / out[8][0], 1),
        "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": round(out[8][0], 4), "dtype": "bf16",
        "data": "synthetic: random weights, uniform random token ids",
        "config": {"model": "Apertus-70B shapes", "layers": cfg.num_hidden_layers, "layers_full": 80, "hidden": H, "heads": nq,
                   "kv_heads": nkv, "head_dim": D, "intermediate": I, "vocab": cfg.vocab_size,
                   "weight_gb": round(engine.weight_bytes() / 1e9, 1), "peaks": pk_source},
        "clocks": clock_info,
        "points": {"decode_b1": round(1000.0 / out[1][0], 2), "decode_b1_ms": round(out[1][0], 4),
                   "decode_b1_frac": round(out[1][1] / pk["hbm_gbs"], 4)},
        "prefill": {"value": round(1024 * 1000.0 / out["prefill_1024"], 1), "tokens": 1024, "ms": round(out["prefill_1024"], 2),
                    "frac": round(flops / (out["prefill_1024"] * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(out[8][1], 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(out[8][1] / pk["hbm_gbs"], 4)}}))
    return 0


def run_sweep(args, pk, pk_source):
    """Apertus-8B sizes at further batch sizes, context lengths and prompt lengths than the headline line: decode steps
    of 1 to 128 sequences after 1,023 to 32,767 cached positions, and prompts of 128 to 8,192 tokens, each with its
    fraction of the measured peak. One line of JSON with two lists."""
    import torch
    from tileinfer_b200.config import ApertusConfig
    from tileinfer_b200.engine import Engine
    cfg_dict = dict(APERTUS_8B, max_position_embeddings=32768 + 256)
    if args.layers:
        cfg_dict["num_hidden_layers"] = args.layers
    cfg = ApertusConfig.from_dict(cfg_dict)
    points = [(1, 1023), (1, 8191), (1, 32767), (4, 1023), (8, 1023), (8, 8191), (8, 32767), (16, 1023), (16, 8191), (32, 1023),
              (32, 8191), (64, 1023), (64, 8191), (128, 1023), (128, 4095)]
    steps, warmup = max(8, min(args.steps, 32)), max(args.warmup, 3)
    room = max(b * (-(-(c + steps + warmup + 8) // 64) * 64) for b, c in points)
    engine = Engine.random(cfg, seed=0, dtype="bfloat16", max_context=32768 + 256, max_seqs=128, max_tokens=room, max_step_tokens=8192)
    clocks = ClockSampler()
    clocks.start()
    decode = []
    for b, c in points:
        pt = decode_point(engine, b, steps, warmup, cfg.vocab_size, pk, cached=c)
        decode.append({"batch": b, "cached": c, "ms": round(pt["ms"], 4), "tok_s": round(pt["value"], 1), "frac": round(pt["frac"], 4)})
    prefill = []
    for tokens in (128, 256, 512, 1024, 2048, 8192):
        ms = time_prefill(engine, tokens, cfg.vocab_size, reps=2)
        flops = flops_prefill(cfg_dict, cfg.num_hidden_layers, tokens)
        prefill.append({"tokens": tokens, "ms": round(ms, 3), "tok_s": round(tokens * 1000.0 / ms, 1),
                        "frac": round(flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                        "weights_frac": round(engine.weight_bytes() / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)})
    clock_info = clocks.stop()
    engine.check_health()
    print(json.dumps({"metric": "decode and prefill at further sizes (Apertus-8B bf16)", "n_gpus": 1, "steps": steps, "warmup": warmup,
                      "dtype": "bf16", "data": "synthetic: random weights, uniform random token ids",
                      "config": {"model": "Apertus-8B shapes", "layers": cfg.num_hidden_layers, "layers_full": 32, "peaks": pk_source},
                      "clocks": clock_info, "decode": decode, "prefill": prefill}))
    return 0


def flops_prefill(cfg, n_layers, tokens):
    H, I, D = cfg["hidden_size"], cfg["intermediate_size"], cfg["head_dim"]
    nq, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    per_layer = 2 * tokens * (H * (nq + 2 * nkv) * D + nq * D * H + 2 * H * I) + 4 * D * nq * tokens * (tokens + 1) // 2
    return n_layers * per_layer + 2 * H * cfg["vocab_size"]


def decode_point(engine, batch, steps, warmup, vocab, pk, count_launches=False, cached=None):
    """One decode measurement: tokens per second, ms per step, the bytes the step has to read (every
    weight once, and the cache of the live sequences) and their rate as a fraction of the HBM peak."""
    ms, kv_positions, launches = time_decode(engine, batch, steps, warmup, vocab, count_launches=count_launches, cached=cached)
    step_bytes = engine.weight_bytes() + kv_positions * engine.kv_bytes_per_position()
    gbs = step_bytes / (ms * 1e-3) / 1e9
    return {"value": batch * 1000.0 / ms, "ms": ms, "bytes": step_bytes, "gbs": gbs, "frac": gbs / pk["hbm_gbs"], "launches": launches}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="run fewer layers than the configuration has (0: all)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"],
                    help="float32: the true 32-bit path (strict 32-bit FMA products) as the headline")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-points", action="store_true", help="only the headline batch (quick checks)")
    ap.add_argument("--preset", default="8b", choices=["8b", "8b-long", "70b", "sweep"],
                    help="8b: the headline line (default); 8b-long: 8 unequal sequences of up to 32,768 positions; "
                         "70b: Apertus-70B sizes, 141 GB of weights")
    args = ap.parse_args(argv)

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "AntoineBut/TileInfer.jl is a Julia package (CUDA.jl + cuTile, sm_89): pip finds neither "
                          "setup.py nor pyproject.toml, and neither Julia nor its packages are on this machine or the network"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures the single-GPU library; --gpus {args.gpus} is not supported (one GPU only)")
        return 2

    import torch
    from tileinfer_b200.config import ApertusConfig
    from tileinfer_b200.engine import Engine

    if args.preset == "8b-long":
        return run_long_context(args, *peaks())
    if args.preset == "70b":
        return run_70b(args, *peaks())
    if args.preset == "sweep":
        return run_sweep(args, *peaks())
    cfg_dict = dict(APERTUS_8B)
    full_layers = cfg_dict["num_hidden_layers"]
    if args.layers:
        cfg_dict["num_hidden_layers"] = args.layers
    cfg = ApertusConfig.from_dict(cfg_dict)
    pk, pk_source = peaks()
    fp32 = args.dtype == "float32"
    vocab = cfg.vocab_size
    batches = sorted({1, args.batch, 64} if not (args.skip_points or fp32) else {args.batch})
    max_batch = max(batches)

    e2e_steps = max(min(args.steps, 16), 8) if fp32 else max(args.steps, 128)
    per_seq = -(-(CACHED + max(e2e_steps, args.steps + args.warmup) + 8) // 64) * 64      # positions a sequence may reach, in whole pages

    def make_engine(dtype):
        return Engine.random(cfg, seed=0, dtype=dtype, max_context=CONTEXT, max_seqs=max_batch,
                             max_tokens=max(max_batch * per_seq, PREFILL_TOKENS + 64), max_step_tokens=PREFILL_TOKENS)

    engine = make_engine(args.dtype)
    prefill_ms = time_prefill(engine, PREFILL_TOKENS, vocab, reps=1 if fp32 else 3)
    points = {}
    for b in batches:
        if b == args.batch:
            continue
        pt = decode_point(engine, b, max(8, args.steps // 2), args.warmup, vocab, pk)
        points.update({f"decode_b{b}": round(pt["value"], 1), f"decode_b{b}_ms": round(pt["ms"], 4),
                       f"decode_b{b}_frac": round(pt["frac"], 4), f"e2e_b{b}": time_e2e(engine, b, e2e_steps, vocab)["value"]})

    clocks = ClockSampler()
    clocks.start()
    head = decode_point(engine, args.batch, args.steps, args.warmup, vocab, pk, count_launches=True)
    clock_info = clocks.stop()
    e2e = time_e2e(engine, args.batch, e2e_steps, vocab, sample_clocks=True)
    e2e.update({"h2d_bytes_per_step": engine.planner.last_upload_bytes, "d2h_bytes_per_step": 4 * args.batch})
    page_size = engine.cache.page_size
    engine.check_health()

    if not fp32 and not args.skip_points:
        # The true 32-bit path at the same sizes: 32-bit weights, activations and cache, strict FMA products.
        del engine
        torch.cuda.empty_cache()
        engine = make_engine("float32")
        pt = decode_point(engine, args.batch, 8, 3, vocab, pk)
        points.update({f"decode_fp32_b{args.batch}": round(pt["value"], 1), f"decode_fp32_b{args.batch}_ms": round(pt["ms"], 4),
                       f"decode_fp32_b{args.batch}_frac": round(pt["frac"], 4)})
        engine.check_health()

    pf_flops = flops_prefill(cfg_dict, cfg.num_hidden_layers, PREFILL_TOKENS)
    pf_peak = FP32_TFLOPS if fp32 else pk["bf16_tflops"]
    name = "fp32" if fp32 else "bf16"
    line = {
        "metric": f"decode tok/s (Apertus-8B {name}, batch {args.batch}, {CACHED} cached positions)", "value": round(head["value"], 1),
        "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(head["ms"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": name,
        "data": "synthetic: random weights, uniform random token ids",
        "config": {"model": "Apertus-8B shapes", "global_batch": args.batch, "seq_len": CONTEXT, "parallelism": "none",
                   "layers": cfg.num_hidden_layers, "layers_full": full_layers, "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "cached_positions": CACHED,
                   "prefill_tokens": PREFILL_TOKENS, "rope_theta": cfg.rope_theta, "page_size": page_size,
                   "l2": "step inputs (16 GB of weights) exceed L2",
                   "peaks": pk_source + (", 32-bit FMA peak nominal" if fp32 else "")},
        "clocks": clock_info,
        "e2e": e2e,
        "gpu_launches": head["launches"] * args.steps,
        "prefill": {"value": round(PREFILL_TOKENS * 1000.0 / prefill_ms, 1), "tokens": PREFILL_TOKENS,
                    "ms": round(prefill_ms, 3), "frac": round(pf_flops / (prefill_ms * 1e-3) / (pf_peak * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(head["gbs"], 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(head["frac"], 4), "bytes": int(head["bytes"])},
        "points": points,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
