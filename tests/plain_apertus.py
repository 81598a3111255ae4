"""Plain, slow Apertus: whole sequences, no cache, one function per part, PyTorch on the CPU.

This file is the oracle of the test-suite. It shares no code with the library under test
(it parses config.json itself and reads safetensors with the ``safetensors`` package), and
every function is written from the formulas of AntoineBut/TileInfer.jl, cited as
``file:line`` within that project.

The reference's own model code (Julia + CUDA.jl + cuTile) can neither be imported nor
compiled on a CPU-only machine without Julia, so this implementation rests on its
formulas. It is anchored once on the reference's committed goldens, which were produced by
Hugging Face transformers' ApertusForCausalLM on a tiny random checkpoint
(scripts/gen_apertus_fixtures.py:116-140): ``tests/test_plain_anchor.py`` replays them.

``dtype`` is ``torch.float32`` (every rounding below is the identity) or
``torch.bfloat16``, in which case values are rounded to bfloat16 at the points where the
reference's kernels round (marked ``rnd``); arithmetic itself always runs in 32-bit.
"""
from __future__ import annotations

import json
import math
import os
from types import SimpleNamespace
from typing import Dict, List, Optional, Sequence

import torch


# ----------------------------------------------------------------------------- configuration
def read_config(c: dict) -> SimpleNamespace:
    """src/config.jl:50-97 (keys and defaults), restricted to Apertus."""
    rope = c.get("rope_parameters")
    theta = c["rope_theta"] if rope is None else rope["rope_theta"]
    scaling = c.get("rope_scaling") if rope is None else rope
    if scaling is not None and scaling.get("rope_type", scaling.get("type", "default")) == "default":
        scaling = None
    heads = c["num_attention_heads"]
    eos = c.get("eos_token_id")
    return SimpleNamespace(
        vocab=c.get("output_vocab_size") or c["vocab_size"], hidden=c["hidden_size"],
        inter=c["intermediate_size"], layers=c["num_hidden_layers"], heads=heads,
        kv_heads=c.get("num_key_value_heads") or heads,
        head_dim=c.get("head_dim") or c["hidden_size"] // heads,
        eps=c["rms_norm_eps"], theta=theta, scaling=scaling,
        max_pos=c["max_position_embeddings"], tied=c.get("tie_word_embeddings", False),
        qk_norm=c.get("qk_norm", False), init_std=c.get("initializer_range", 0.02),
        eos=[] if eos is None else [eos] if isinstance(eos, int) else list(eos),
    )


def load_folder(model_dir: str):
    """config + {name: float32 tensor} of a model folder, through the safetensors package."""
    from safetensors import safe_open
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = read_config(json.load(f))
    weights = {}
    for fn in sorted(os.listdir(model_dir)):
        if fn.endswith(".safetensors"):
            with safe_open(os.path.join(model_dir, fn), "pt") as f:
                for k in f.keys():
                    weights[k] = f.get_tensor(k).float()
    return cfg, weights


def rnd(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """Round to the storage type and come back to 32-bit."""
    return x if dtype == torch.float32 else x.to(dtype).float()


# ----------------------------------------------------------------------------- parts
def embed(table: torch.Tensor, ids: Sequence[int]) -> torch.Tensor:
    """x[t] = E[ids[t]], 0-based ids, no scaling (src/ops/reference.jl:10)."""
    return table[torch.as_tensor(list(ids), dtype=torch.long)]


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, dtype: torch.dtype) -> torch.Tensor:
    """Normalise in 32-bit, round, then scale by w in the storage type (src/ops/reference.jl:17-21)."""
    inv_rms = 1.0 / torch.sqrt(x.pow(2).sum(-1, keepdim=True) / x.shape[-1] + torch.tensor(eps, dtype=torch.float32))
    return rnd(w * rnd(x * inv_rms, dtype), dtype)


def linear(x: torch.Tensor, W: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """y = x Wᵀ for W [out, in], 32-bit accumulation, one rounding (src/ops/reference.jl:23-26)."""
    return rnd(x @ W.t(), dtype)


def inverse_frequencies(cfg) -> torch.Tensor:
    """f_i = 1/theta^(2i/D) in 32-bit, then llama3 scaling per frequency (src/model/rope.jl:15-38)."""
    D = cfg.head_dim
    inv = 1.0 / (torch.tensor(float(cfg.theta), dtype=torch.float32) **
                 (torch.arange(0, D, 2, dtype=torch.float32) / torch.tensor(float(D), dtype=torch.float32)))
    s = cfg.scaling
    if s is None:
        return inv
    f32 = lambda v: torch.tensor(float(v), dtype=torch.float32)
    factor, low, high = f32(s["factor"]), f32(s["low_freq_factor"]), f32(s["high_freq_factor"])
    old = f32(s["original_max_position_embeddings"])
    wavelen = 2.0 * f32(math.pi) / inv
    smooth = (old / wavelen - low) / (high - low)
    mid = (1 - smooth) * inv / factor + smooth * inv
    return torch.where(wavelen < old / high, inv, torch.where(wavelen > old / low, inv / factor, mid))


def rope_tables(cfg, positions: torch.Tensor, dtype: torch.dtype):
    """angle = fp32(p)·f in 32-bit; cos/sin in 64-bit of that angle, rounded to 32-bit then to the
    storage type; both halves share the angles (src/model/rope.jl:40-45)."""
    ang = positions.to(torch.float32)[:, None] * inverse_frequencies(cfg)[None, :]
    ang = torch.cat([ang, ang], -1)
    return rnd(ang.double().cos().float(), dtype), rnd(ang.double().sin().float(), dtype)


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """Rotate-half pairing i <-> i + D/2, each operation rounded (src/ops/reference.jl:32-39).
    x is [n, heads, D]; cos/sin are [n, D]."""
    half = x.shape[-1] // 2
    rotated = torch.cat([-x[..., half:], x[..., :half]], -1)
    return rnd(rnd(x * cos[:, None, :], dtype) + rnd(rotated * sin[:, None, :], dtype), dtype)


def xielu_scalars(alpha_p_raw, alpha_n_raw, beta_raw, eps_raw, dtype: torch.dtype):
    """beta = T(beta); alpha_p = T(softplus(raw)); alpha_n = T(beta + T(softplus(raw))); eps = T(eps);
    softplus = log1p(exp(x)) on the 32-bit value (src/hub/loader.jl:193-202)."""
    sp = lambda t: torch.log1p(torch.exp(t.float().reshape(())))
    beta = rnd(beta_raw.float().reshape(()), dtype)
    return SimpleNamespace(alpha_p=rnd(sp(alpha_p_raw), dtype), alpha_n=rnd(beta + rnd(sp(alpha_n_raw), dtype), dtype),
                           beta=beta, eps=rnd(eps_raw.float().reshape(()), dtype))


def xielu(x: torch.Tensor, a, dtype: torch.dtype) -> torch.Tensor:
    """x > 0 ? alpha_p·x·x + beta·x : (expm1(min(x, eps)) − x)·alpha_n + beta·x, rounded after every
    operation, expm1 evaluated in 32-bit (src/ops/reference.jl:49-56)."""
    r = lambda t: rnd(t, dtype)
    bx = r(a.beta * x)
    pos = r(r(r(a.alpha_p * x) * x) + bx)
    neg = r(r(r(r(torch.expm1(torch.minimum(x, a.eps))) - x) * a.alpha_n) + bx)
    return torch.where(x > 0, pos, neg)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, dtype: torch.dtype,
              start: int = 0, window: int = 0) -> torch.Tensor:
    """Causal grouped-query attention over whole sequences.

    q [n, nq, D] are the queries at positions start..start+n-1; k, v [start+n, nkv, D] are all
    keys/values. Query head h reads KV head h div g (src/ops/reference.jl:108-112); key i is
    visible to the query at position p iff i <= p (reference.jl:98-107). Scores and softmax
    stay in 32-bit; P is rounded only for the PV product, the sum is 32-bit, O is rounded
    (the kernels' convention, src/ops/tile/attention.jl:1-3, 34-59). ``window`` > 0 lets a query
    see only its last ``window`` keys, itself included; the reference refuses such models
    (src/config.jl:60-62), the library's cache groups with a window are tested with it."""
    n, nq, D = q.shape
    total, nkv, _ = k.shape
    g = nq // nkv
    kk = k.repeat_interleave(g, 1)
    vv = v.repeat_interleave(g, 1)
    s = torch.einsum("qhd,khd->hqk", q, kk) * torch.tensor(scale, dtype=torch.float32)
    qpos = torch.arange(start, start + n)[:, None]
    kpos = torch.arange(total)[None, :]
    s = s.masked_fill((kpos > qpos)[None], float("-inf"))
    if window:
        s = s.masked_fill((kpos <= qpos - window)[None], float("-inf"))
    e = torch.exp(s - s.max(-1, keepdim=True).values)
    o = torch.einsum("hqk,khd->qhd", rnd(e, dtype), vv) / e.sum(-1).t()[:, :, None]
    return rnd(o, dtype)


def attention_block(h, W, p, cfg, positions, dtype, window: int = 0):
    """q/k/v projections, per-head q/k RMSNorm before RoPE, attention, output projection
    (src/model/decoder.jl:176-180; src/ops/interface.jl:161-177)."""
    n = h.shape[0]
    D = cfg.head_dim
    q = linear(h, W[p + "self_attn.q_proj.weight"], dtype).view(n, cfg.heads, D)
    k = linear(h, W[p + "self_attn.k_proj.weight"], dtype).view(n, cfg.kv_heads, D)
    v = linear(h, W[p + "self_attn.v_proj.weight"], dtype).view(n, cfg.kv_heads, D)
    if cfg.qk_norm:
        q = rmsnorm(q, rnd(W[p + "self_attn.q_norm.weight"], dtype), cfg.eps, dtype)
        k = rmsnorm(k, rnd(W[p + "self_attn.k_norm.weight"], dtype), cfg.eps, dtype)
    cos, sin = rope_tables(cfg, positions, dtype)
    q, k = rope(q, cos, sin, dtype), rope(k, cos, sin, dtype)
    o = attention(q, k, v, 1.0 / math.sqrt(D), dtype, window=window)          # scale fixed in code: decoder.jl:169
    return linear(o.reshape(n, cfg.heads * D), W[p + "self_attn.o_proj.weight"], dtype)


def feed_forward(h, W, p, dtype):
    """up -> xIELU -> down, no gate, no biases (src/model/decoder.jl:183-189)."""
    a = xielu_scalars(W[p + "mlp.act_fn.alpha_p"], W[p + "mlp.act_fn.alpha_n"], W[p + "mlp.act_fn.beta"],
                      W[p + "mlp.act_fn.eps"], dtype)
    return linear(xielu(linear(h, W[p + "mlp.up_proj.weight"], dtype), a, dtype), W[p + "mlp.down_proj.weight"], dtype)


def forward(cfg, W: Dict[str, torch.Tensor], ids: Sequence[int], dtype: torch.dtype = torch.float32,
            windows: Sequence[int] = ()) -> torch.Tensor:
    """Logits [n, vocab] (32-bit) of one whole sequence (src/model/decoder.jl:165-196). ``windows``:
    an attention window for each layer (0: none), see :func:`attention`."""
    W = {k: (rnd(v, dtype) if v.dim() >= 1 and v.numel() > 1 else v) for k, v in W.items()}
    positions = torch.arange(len(ids))
    x = embed(W["model.embed_tokens.weight"][: cfg.vocab], ids)
    for l in range(cfg.layers):
        p = f"model.layers.{l}."
        h = rmsnorm(x, W[p + "attention_layernorm.weight"], cfg.eps, dtype)
        window = windows[l] if windows else 0
        x = rnd(x + attention_block(h, W, p, cfg, positions, dtype, window), dtype)      # src/ops/tile/norm.jl:53-55
        h = rmsnorm(x, W[p + "feedforward_layernorm.weight"], cfg.eps, dtype)
        x = rnd(x + feed_forward(h, W, p, dtype), dtype)
    h = rmsnorm(x, W["model.norm.weight"], cfg.eps, dtype)
    head = W["model.embed_tokens.weight"][: cfg.vocab] if cfg.tied else W["lm_head.weight"]
    return linear(h, head, dtype)                                                # rounded, then 32-bit out


# ----------------------------------------------------------------------------- random weights
def random_normal(seed: int, name: str, count: int):
    """The library's random-weights function, restated: z_i = f(seed, name, i), i < count, as float32.

    The reference has no random-weights mode (its only random model is a fixture script,
    scripts/gen_apertus_fixtures.py:80-96); the function is this library's own, built on the reference's
    integer mix (src/engine/sampler.jl:34-47): keys k0 = mix32(mix32(seed) xor fnv1a(name)),
    k1 = mix32(k0 + 0x9E3779B9); a = mix32(k0 xor i) >> 8, b = mix32(k1 xor i) >> 8; Box-Muller
    z = sqrt(-2 ln((a + 1) 2^-24)) cos(2 pi b 2^-24), with the logarithm (2 atanh series of the mantissa
    brought into (sqrt 1/2, sqrt 2]) and the cosine (octants of b, Taylor series on [0, pi/4]) spelled out
    in single 32-bit operations, so that every machine gets the same bits."""
    import numpy as np
    f32, u32 = np.float32, np.uint32
    name_hash = 0x811C9DC5
    for byte in name.encode():
        name_hash = ((name_hash ^ byte) * 0x01000193) % 2 ** 32
    k0 = mix32(mix32(seed % 2 ** 32) ^ name_hash)
    k1 = mix32((k0 + 0x9E3779B9) % 2 ** 32)

    def mix(x):
        x = (x ^ (x >> u32(16))) * u32(0x7FEB352D)
        x = (x ^ (x >> u32(15))) * u32(0x846CA68B)
        return x ^ (x >> u32(16))

    def series(coefficients, y):
        acc = np.full(y.shape, f32(coefficients[0]), f32)
        for c in coefficients[1:]:
            acc = acc * y
            acc = acc + f32(c)
        return acc

    i = np.arange(count, dtype=u32)
    a, b = mix(i ^ u32(k0)) >> u32(8), mix(i ^ u32(k1)) >> u32(8)
    mant, expo = np.frexp((a + u32(1)).astype(f32))            # n = mant 2^expo, mant in [0.5, 1)
    m, e = mant * f32(2), expo.astype(np.int32) - 1              # m in [1, 2)
    fold = m > f32(math.sqrt(2.0))
    m, e = np.where(fold, m * f32(0.5), m), e + fold
    s = (m - f32(1)) / (m + f32(1))
    ln_u = (e - 24).astype(f32) * f32(math.log(2.0)) + s * series([2 / 9, 2 / 7, 2 / 5, 2 / 3, 2.0], s * s)
    radius = np.sqrt(f32(-2) * ln_u)
    octant = b >> u32(21)
    frac = (b % u32(1 << 21)).astype(f32) * f32(2.0 ** -21)
    x = np.where(octant % 2 == 1, f32(1) - frac, frac) * f32(math.pi / 4)
    sin_x = x * series([1 / 362880, -1 / 5040, 1 / 120, -1 / 6, 1.0], x * x)
    cos_x = series([-1 / 3628800, 1 / 40320, -1 / 720, 1 / 24, -0.5, 1.0], x * x)
    c = np.where(np.isin(octant, (1, 2, 5, 6)), sin_x, cos_x)
    c = np.where(np.isin(octant, (2, 3, 4, 5)), -c, c)
    return radius * c


def random_weights(cfg, seed: int, dtype: torch.dtype = torch.bfloat16) -> Dict[str, torch.Tensor]:
    """The model that the library's random-weights mode makes for ``cfg`` and ``seed``, as 32-bit tensors
    holding values rounded to ``dtype``: matrices N(0, std), norm weights 1 + N(0, std), raw xIELU alphas
    log(e^0.8 - 1) + N(0, 0.05), beta 0.5, eps -1e-6; value = mean + z std in 32-bit."""
    import numpy as np
    H, D, std = cfg.hidden, cfg.head_dim, cfg.init_std
    shapes = {"model.embed_tokens.weight": ((cfg.vocab, H), 0.0, std), "model.norm.weight": ((H,), 1.0, std)}
    if not cfg.tied:
        shapes["lm_head.weight"] = ((cfg.vocab, H), 0.0, std)
    raw_alpha = math.log(math.expm1(0.8))
    consts = {}
    for l in range(cfg.layers):
        p = f"model.layers.{l}."
        shapes.update({
            p + "attention_layernorm.weight": ((H,), 1.0, std), p + "feedforward_layernorm.weight": ((H,), 1.0, std),
            p + "self_attn.q_proj.weight": ((cfg.heads * D, H), 0.0, std),
            p + "self_attn.k_proj.weight": ((cfg.kv_heads * D, H), 0.0, std),
            p + "self_attn.v_proj.weight": ((cfg.kv_heads * D, H), 0.0, std),
            p + "self_attn.o_proj.weight": ((H, cfg.heads * D), 0.0, std),
            p + "mlp.up_proj.weight": ((cfg.inter, H), 0.0, std), p + "mlp.down_proj.weight": ((H, cfg.inter), 0.0, std),
            p + "mlp.act_fn.alpha_p": ((1,), raw_alpha, 0.05), p + "mlp.act_fn.alpha_n": ((1,), raw_alpha, 0.05)})
        if cfg.qk_norm:
            shapes.update({p + "self_attn.q_norm.weight": ((D,), 1.0, std), p + "self_attn.k_norm.weight": ((D,), 1.0, std)})
        consts.update({p + "mlp.act_fn.beta": 0.5, p + "mlp.act_fn.eps": -1e-6})
    out = {}
    for name, (shape, mean, sd) in shapes.items():
        z = random_normal(seed, name, int(np.prod(shape)))
        out[name] = rnd(torch.from_numpy(np.float32(mean) + z * np.float32(sd)).reshape(shape), dtype)
    for name, value in consts.items():
        out[name] = rnd(torch.tensor(value, dtype=torch.float32), dtype)
    return out


# ----------------------------------------------------------------------------- sampling (host rule)
def mix32(x: int) -> int:
    """lowbias32 (src/engine/sampler.jl:34-38)."""
    x &= 0xFFFFFFFF
    x = ((x ^ (x >> 16)) * 0x7FEB352D) & 0xFFFFFFFF
    x = ((x ^ (x >> 15)) * 0x846CA68B) & 0xFFFFFFFF
    return x ^ (x >> 16)


def sampling_uniform(seed: int, counter: int) -> float:
    """u in [0,1): 24 bits of mix32(mix32(seed) xor counter) (src/engine/sampler.jl:46-47)."""
    return float((mix32(mix32(seed) ^ (counter & 0xFFFFFFFF)) >> 8)) * 2.0 ** -24


def top_candidates(logits: torch.Tensor, k: int) -> List[int]:
    """Ids of the k largest logits, best first, ties to the smaller id (src/engine/sampler.jl:52-58)."""
    order = sorted(range(len(logits)), key=lambda i: (-float(logits[i]), i))
    return order[:k]


def filtered_dist(logits: torch.Tensor, temperature: float, top_k: int, top_p: float):
    """Temperature, then top-k, then top-p over the renormalised survivors, best first
    (src/engine/sampler.jl:68-81)."""
    if temperature == 0:
        return [int(torch.argmax(logits))], [1.0]
    V = len(logits)
    ids = top_candidates(logits, V if top_k == 0 else min(top_k, V))
    scaled = [float(logits[i]) / temperature for i in ids]
    probs = [math.exp(s - scaled[0]) for s in scaled]
    total = sum(probs)
    probs = [p / total for p in probs]
    if top_p < 1:
        cum, n = 0.0, len(probs)
        for j, p in enumerate(probs):
            cum += p
            if cum >= top_p:
                n = j + 1
                break
        sub = sum(probs[:n])
        ids, probs = ids[:n], [p / sub for p in probs[:n]]
    return ids, probs


def pick(weights: Sequence[float], u: float) -> int:
    """First entry with positive weight whose cumulative weight reaches u × total
    (src/engine/sampler.jl:88-91)."""
    total = sum(weights)
    cum, last = 0.0, 0
    for i, w in enumerate(weights):
        cum += w
        if w > 0:
            last = i
            if cum >= u * total:
                return i
    return last


def sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, u: float) -> int:
    """src/engine/sampler.jl:99-102."""
    ids, probs = filtered_dist(logits, temperature, top_k, top_p)
    return ids[pick(probs, u)]


def generate(cfg, W, prompt: Sequence[int], max_new_tokens: int, dtype=torch.float32, temperature: float = 0.0,
             top_k: int = 0, top_p: float = 1.0, seed: int = 0, stop_ids: Sequence[int] = ()) -> List[int]:
    """The loop of src/engine/generate.jl:43-56 by full recomputation: sample, stop check (the stop
    token is not emitted), append, budget check."""
    ids = list(prompt)
    out: List[int] = []
    for counter in range(max_new_tokens):
        logits = forward(cfg, W, ids, dtype)[-1]
        t = sample(logits, temperature, top_k, top_p, sampling_uniform(seed, counter))
        if t in stop_ids:
            break
        out.append(t)
        ids.append(t)
    return out
