"""Tensor-level wrappers of the CUDA kernels.

Each function checks devices, element types and layouts, then launches on the current
stream; outputs are passed in by the caller, so a step made of these calls allocates
nothing and can be captured in a CUDA graph.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import library as _library

from .library import KernelError, check, lib

F32, BF16 = 0, 1
EPI_NONE, EPI_XIELU, EPI_F32_OUT = 0, 1, 2
MAX_HEAD_DIM = 512      # the largest head the attention kernels take (csrc/attention_inputs.cu, csrc/attention_plain.cu)


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, not {dtype}")


def _stream() -> int:
    return _library.current_stream()


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, name: str, dtype=None, contiguous=True):
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


def random_normal(out, k0: int, k1: int, mean: float, std: float, first: int = 0):
    """out.flat[j] = mean + std * z(first + j) of the counter-based generator with keys (k0, k1)."""
    _need(out, "out")
    check(lib().ti_random_normal(out.data_ptr(), dtype_code(out.dtype), out.numel(), first, k0, k1, mean, std, _stream()),
          "random_normal")


def embed(out, table, ids, status):
    _need(out, "out"); _need(table, "table", out.dtype); _need(ids, "ids", torch.int32); _need(status, "status", torch.int32)
    n, hidden = out.shape
    check(lib().ti_embed(out.data_ptr(), table.data_ptr(), ids.data_ptr(), n, hidden, table.shape[0],
                         dtype_code(out.dtype), status.data_ptr(), _stream()), "embed")


def gather_rows(out, x, idx):
    _need(out, "out"); _need(x, "x", out.dtype); _need(idx, "idx", torch.int32)
    check(lib().ti_gather_rows(out.data_ptr(), x.data_ptr(), idx.data_ptr(), out.shape[0], out.shape[1],
                               dtype_code(out.dtype), _stream()), "gather_rows")


def xielu(out, x, alpha_p, alpha_n, beta, eps):
    _need(out, "out"); _need(x, "x", out.dtype)
    check(lib().ti_xielu(out.data_ptr(), x.data_ptr(), x.numel(), alpha_p, alpha_n, beta, eps,
                         dtype_code(out.dtype), _stream()), "xielu")


def rmsnorm(out, x, w, eps):
    _need(out, "out"); _need(x, "x", out.dtype); _need(w, "w", out.dtype)
    size = x.shape[-1]
    check(lib().ti_rmsnorm(out.data_ptr(), x.data_ptr(), w.data_ptr(), x.numel() // size, size, eps,
                           dtype_code(out.dtype), _stream()), "rmsnorm")


def add_rmsnorm(x, delta, w, h, eps, partials=None):
    """x <- x + delta (or the sum of 32-bit ``partials`` [s, n, size]); h <- RMSNorm(x)·w."""
    _need(x, "x"); _need(w, "w", x.dtype); _need(h, "h", x.dtype)
    n, size = x.shape
    if partials is not None:
        _need(partials, "partials", torch.float32)
        s = partials.shape[0]
        check(lib().ti_add_rmsnorm(x.data_ptr(), None, partials.data_ptr(), s, partials.stride(0), w.data_ptr(),
                                   h.data_ptr(), n, size, eps, dtype_code(x.dtype), _stream()), "add_rmsnorm")
    else:
        _need(delta, "delta", x.dtype)
        check(lib().ti_add_rmsnorm(x.data_ptr(), delta.data_ptr(), None, 0, 0, w.data_ptr(), h.data_ptr(), n, size,
                                   eps, dtype_code(x.dtype), _stream()), "add_rmsnorm")


def add(x, delta):
    _need(x, "x"); _need(delta, "delta", x.dtype)
    check(lib().ti_add(x.data_ptr(), delta.data_ptr(), x.numel(), dtype_code(x.dtype), _stream()), "add")


def attention_inputs(qkv, q_out, k_cache, v_cache, q_norm_w, k_norm_w, eps, rotation, positions, slots,
                     nq, nkv, head_dim, page_size, write_kv=True):
    """qkv [n, (nq + 2 nkv) D] -> q_out [n, nq, D]; k and v rows into the pools at ``slots``. ``qkv`` may
    also be the 32-bit partial sums [s, n, features] of a projection that was split over k. ``rotation``:
    None, or a record with ``cos_sin`` [positions, rotary_dim / 2, 2] float32, ``rotary_dim`` and
    ``interleaved`` (see ``parts.base.Rotation``)."""
    cos_sin = rotation.cos_sin if rotation is not None else None
    rotary, interleaved = (int(rotation.rotary_dim), int(bool(rotation.interleaved))) if rotation is not None else (0, 0)
    if rotation is not None and (rotary < 2 or rotary % 2 or rotary > head_dim or cos_sin.shape[1] * 2 != rotary):
        raise KernelError(f"rotation over {rotary} of {head_dim} elements with a table of {tuple(cos_sin.shape)}")
    _need(qkv, "qkv", contiguous=False); _need(q_out, "q_out")
    _need(positions, "positions", torch.int32)
    if qkv.stride(-1) != 1:
        raise KernelError("qkv rows must be dense")
    if write_kv:
        _need(k_cache, "k_cache", q_out.dtype); _need(v_cache, "v_cache", q_out.dtype); _need(slots, "slots", torch.int32)
    if cos_sin is not None:
        _need(cos_sin, "cos_sin", torch.float32)
    if qkv.dim() == 3:
        _need(qkv, "partial sums", torch.float32)
        args = (None, qkv.stride(1), qkv.data_ptr(), qkv.shape[0], qkv.stride(0))
        n = qkv.shape[1]
    else:
        if qkv.dtype != q_out.dtype:
            raise KernelError(f"qkv must be {q_out.dtype}")
        args = (qkv.data_ptr(), qkv.stride(0), None, 0, 0)
        n = qkv.shape[0]
    check(lib().ti_attention_inputs(*args, q_out.data_ptr(), _ptr(k_cache), _ptr(v_cache),
                                    _ptr(q_norm_w), _ptr(k_norm_w), eps, _ptr(cos_sin), rotary, interleaved, positions.data_ptr(),
                                    _ptr(slots), n, nq, nkv, head_dim, page_size, int(write_kv),
                                    dtype_code(q_out.dtype), _stream()), "attention_inputs")


def attention_plain(out, q, k_cache, v_cache, block_table, tok_slot, positions, scale, nq, nkv, head_dim,
                    page_size, window=0):
    _need(out, "out"); _need(q, "q", out.dtype); _need(k_cache, "k_cache", out.dtype); _need(v_cache, "v_cache", out.dtype)
    _need(block_table, "block_table", torch.int32); _need(tok_slot, "tok_slot", torch.int32)
    _need(positions, "positions", torch.int32)
    check(lib().ti_attention_plain(out.data_ptr(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                   block_table.data_ptr(), block_table.stride(0), tok_slot.data_ptr(),
                                   positions.data_ptr(), scale, q.shape[0], nq, nkv, head_dim, page_size, window or 0,
                                   dtype_code(out.dtype), _stream()), "attention_plain")


def gemm_plain(y, x, w, epilogue=EPI_NONE, act=(0.0, 0.0, 0.0, 0.0)):
    """y[n, out] = x[n, in] · w[out, in]ᵀ on the CUDA cores in 32-bit arithmetic."""
    _need(x, "x", contiguous=False); _need(w, "w", x.dtype); _need(y, "y", contiguous=False)
    n, k = x.shape
    out = w.shape[0]
    if w.shape[1] != k or y.shape[0] != n or y.shape[1] != out or x.stride(1) != 1 or y.stride(1) != 1:
        raise KernelError(f"gemm: shapes x {tuple(x.shape)}, w {tuple(w.shape)}, y {tuple(y.shape)} do not fit")
    want = torch.float32 if epilogue == EPI_F32_OUT else x.dtype
    if y.dtype != want:
        raise KernelError(f"gemm: output must be {want}")
    check(lib().ti_gemm_plain(y.data_ptr(), y.stride(0), x.data_ptr(), x.stride(0), w.data_ptr(), n, out, k, epilogue,
                              act[0], act[1], act[2], act[3], dtype_code(x.dtype), _stream()), "gemm_plain")


_argmax_ws = {}


def argmax_workspace(rows: int, vocab: int, device):
    """(values, ids, counters) for ``argmax`` over ``rows`` rows: one per device, grown on demand. The
    counters start at zero and every launch leaves them at zero."""
    chunks = lib().ti_argmax_chunks(vocab)
    key = str(device)
    ws = _argmax_ws.get(key)
    if ws is None or ws[0].numel() < rows * chunks or ws[2].numel() < rows:
        n = max(rows, 64)
        ws = _argmax_ws[key] = (torch.empty(n * 256, dtype=torch.float32, device=device),
                                torch.empty(n * 256, dtype=torch.int32, device=device),
                                torch.zeros(n, dtype=torch.int32, device=device))
    return ws


def argmax(logits, out, workspace=None, also=None):
    """out[row] = the largest logit's id, ties to the smaller id; ``also``: a second int32 vector that gets the same
    tokens (the next step's token ids)."""
    _need(logits, "logits", torch.float32, contiguous=False); _need(out, "out", torch.int32)
    val, idx, cnt = workspace or argmax_workspace(logits.shape[0], logits.shape[1], logits.device)
    check(lib().ti_argmax(logits.data_ptr(), logits.stride(0), logits.shape[0], logits.shape[1], out.data_ptr(), _ptr(also),
                          val.data_ptr(), idx.data_ptr(), cnt.data_ptr(), _stream()), "argmax")


def sample(logits, out, temperature, top_k, top_p, seeds, counters, also=None, cluster_blocks=0):
    """``cluster_blocks``: how many blocks share a row (1, 2, 4 or 8); 0 lets the library choose from the number of
    rows and the vocabulary. The token does not depend on it."""
    _need(logits, "logits", torch.float32, contiguous=False); _need(out, "out", torch.int32)
    _need(seeds, "seeds", torch.int32); _need(counters, "counters", torch.int32)
    check(lib().ti_sample_shared(logits.data_ptr(), logits.stride(0), logits.shape[0], logits.shape[1], temperature, top_k,
                                 top_p, seeds.data_ptr(), counters.data_ptr(), out.data_ptr(), _ptr(also), cluster_blocks,
                                 _stream()), "sample")
