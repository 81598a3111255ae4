"""Choice of the bfloat16 kernels. Each function returns None/False when the sizes are
outside what the fast kernels take, in which case the caller runs the plain CUDA-core
kernel instead (same result up to rounding); it never returns a wrong result."""
from __future__ import annotations

import torch

from . import library as _library

from . import ops
from .library import KernelError, add_launches, check, lib

GEMV_MAX_TOKENS = 8          # from 9 tokens on the tensor-core product is faster (measured per layer: 151 against 162 us at 12 tokens)
_sm_count = 0


def sm_count() -> int:
    """Streaming multiprocessors of the device, asked once (148, a B200, where no device answers: the
    plans below can be computed and tested without one)."""
    global _sm_count
    if not _sm_count:
        _sm_count = int(_library.declare("ti_sm_count", [])())
    return _sm_count


def _stream() -> int:
    return _library.current_stream()


def gemv_splits(out_features: int, in_features: int) -> int:
    """How many slices of k a decode product is cut into when its consumer can add partial sums: only
    products with so few output rows that their blocks (16 rows each) would leave SMs idle. (With one block
    per SM or more, unsplit is fastest: the down projection of 8 tokens streams at 5.7 TB/s unsplit, 5.4
    in three slices, and its consumer then reads one rounded result instead of three partial sums.)"""
    row_blocks = -(-out_features // 16)
    if row_blocks >= sm_count():
        return 1
    return max(1, min(8, (2 * sm_count()) // row_blocks, in_features // 1024))


def linear(lin, x, out, epilogue, act, allow_partials=False):
    """Returns the tensor that holds the result (``out``, or 32-bit partial sums [s, n, out] when
    ``allow_partials``), or None when no fast kernel takes these sizes."""
    n, k = x.shape
    w = lin.weight
    if x.dtype != torch.bfloat16 or n == 0:
        return None
    if n <= GEMV_MAX_TOKENS and k % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0:
        splits = gemv_splits(lin.out_features, k) if (allow_partials and epilogue == ops.EPI_NONE) else 1
        if splits > 1:
            partials = lin.rt.buffer("linear.partials", (splits, n, lin.out_features), torch.float32)
            check(lib().ti_gemv_bf16(partials.data_ptr(), lin.out_features, x.data_ptr(), x.stride(0), w.data_ptr(), n,
                                     lin.out_features, k, splits, 3, 0.0, 0.0, 0.0, 0.0, _stream()), "gemv_bf16")
            return partials
        check(lib().ti_gemv_bf16(out.data_ptr(), out.stride(0), x.data_ptr(), x.stride(0), w.data_ptr(), n,
                                 lin.out_features, k, 1, epilogue, act[0], act[1], act[2], act[3], _stream()), "gemv_bf16")
        return out
    if k % 8 == 0 and k >= 8 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0:
        return _tcgen05(lin, x, out, epilogue, act, allow_partials)
    return None


_status = None


def status_word() -> torch.Tensor:
    """Device word that kernels with bounded waits write a code to when a wait runs out."""
    global _status
    if _status is None:
        _status = torch.zeros(1, dtype=torch.int32, device="cuda")
    return _status


def check_status() -> None:
    """Raise if a kernel gave up on a wait since the last check (costs one device read)."""
    if _status is not None:
        code = int(_status.item())
        if code:
            _status.zero_()
            raise KernelError(f"a tensor-core kernel gave up waiting on a barrier (waits {[i for i in range(31) if code >> i & 1]}); its results are invalid")


def tc_splits(out_features: int, in_features: int, n: int) -> int:
    """How many slices of k the tensor-core product of a decode batch is cut into when its consumer can
    add partial sums: as many as fill the device's block slots (two per SM for token tiles of up to 64), at
    most 8, each at least 512 of k. Measured at 64 tokens: down projection 46 us in 3 slices, 35 us in 8;
    o 17 us in 2, 11 us in 8."""
    if n > 256:
        # A prompt of a few hundred tokens: tiles of 256 weight rows x 256 tokens on SM pairs. A product with few output
        # rows has fewer of them than there are pairs (the down projection of 512 tokens: 32 tiles for 74 pairs) and is
        # cut over k into the number of slices (up to 4, each at least 1,024 of k) that takes the fewest rounds of the pairs.
        tiles = -(-out_features // 256) * -(-n // 256)
        pairs = max(1, sm_count() // 2)
        tile_us = in_features * 0.00585                  # 256 x 256 x k on two SMs at 11.2 TFLOP/s each
        whole = -(-tiles // pairs) * tile_us
        best, best_time = 1, 0.9 * whole                 # an estimate: cut only for a tenth or more (a slice that was not
        for s in range(2, min(4, in_features // 1024) + 1):          # worth it: 70B's down projection of 1,024 tokens, +4 % a layer)
            # rounds of the pairs, each 1/s as long; the slices' 32-bit sums are written, and read again by the consumer
            time = -(-tiles * s // pairs) * tile_us / s + s * n * out_features * 8 / 5e6
            if time < best_time - 1e-9:
                best, best_time = s, time
        return best
    tiles = -(-out_features // 128) * -(-n // (256 if n > 128 else 128 if n > 64 else 64 if n > 32 else 32))
    slots = sm_count() * (2 if n <= 64 else 1)
    if tiles >= slots:
        return 1
    return max(1, min(8, slots // tiles, (in_features // 64) // 8))


# The product with the tokens in the tensor-memory lanes (gemm_tcgen05_decode.cu) takes up to 256 tokens (two halves of
# 128 from 129 on: a prompt of 256 tokens runs its up projection in 55 us there instead of 67 us in two rounds of SM pairs).
# The engine uses it from 65 tokens on for the products whose k cannot be cut (activation or logits
# epilogue). Measured inside a decode step of Apertus-8B layers against the 128-row kernel: at 128 tokens
# the up projection takes 41.6 us instead of 58.0 (its 168 tiles of 128 rows need a second round of blocks;
# 135 tiles of 160 rows do not), the layer 229 us instead of 246; at 96 tokens the step is 4 % shorter. Up
# to 64 tokens the 128-row kernel with two blocks per SM is faster inside the step (1,495 against 1,537 us
# for 8 layers at 48 tokens), and products that may be cut over k are no faster here, while more slices cost
# their consumer more (residual add + norm of 128 tokens: 8 us with 4 slices, 15 us with 7).
DECODE_PRODUCT_MIN_TOKENS = 65
DECODE_PRODUCT_MAX_TOKENS = 256
_plans = {}


def decode_product_plan(n: int, out_features: int, in_features: int, max_splits: int):
    """(weight rows per tile, k slices) of the decode-batch product, as its own cost model chooses them."""
    key = (n, out_features, in_features, max_splits)
    plan = _plans.get(key)
    if plan is None:
        import ctypes
        nt, splits = ctypes.c_int(), ctypes.c_int()
        check(lib().ti_gemm_tcgen05_decode_plan(n, out_features, in_features, max_splits, sm_count(), ctypes.byref(nt),
                                                ctypes.byref(splits)), "gemm_tcgen05_decode_plan")
        plan = _plans[key] = (nt.value, splits.value)
    return plan


def _tcgen05_decode(lin, x, out, epilogue, act, allow_partials):
    n, k = x.shape
    w = lin.weight
    may_split = allow_partials and epilogue == ops.EPI_NONE
    nt, splits = decode_product_plan(n, lin.out_features, k, 8 if may_split else 1)
    if splits > 1:
        y = lin.rt.buffer("linear.partials", (splits, n, lin.out_features), torch.float32)
        ldy, epilogue, act = lin.out_features, 3, (0.0, 0.0, 0.0, 0.0)
    else:
        y, ldy = out, out.stride(0)
    rc = lib().ti_gemm_tcgen05_decode(y.data_ptr(), ldy, x.data_ptr(), x.stride(0), w.data_ptr(), n, lin.out_features, k, nt,
                                      splits, epilogue, act[0], act[1], act[2], act[3], status_word().data_ptr(), _stream())
    if rc == 2:
        return None
    check(rc, "gemm_tcgen05_decode")
    return y


def _tcgen05(lin, x, out, epilogue, act, allow_partials):
    n, k = x.shape
    w = lin.weight
    may_split = allow_partials and epilogue == ops.EPI_NONE
    if DECODE_PRODUCT_MIN_TOKENS <= n <= DECODE_PRODUCT_MAX_TOKENS and not may_split:
        y = _tcgen05_decode(lin, x, out, epilogue, act, allow_partials)
        if y is not None:
            return y
    st = status_word()
    splits = tc_splits(lin.out_features, k, n) if (allow_partials and epilogue == ops.EPI_NONE) else 1
    if splits > 1:
        partials = lin.rt.buffer("linear.partials", (splits, n, lin.out_features), torch.float32)
        rc = lib().ti_gemm_tcgen05(partials.data_ptr(), lin.out_features, x.data_ptr(), x.stride(0), w.data_ptr(), n,
                                   lin.out_features, k, splits, 3, 0.0, 0.0, 0.0, 0.0, st.data_ptr(), _stream())
        if rc == 2:
            return None
        check(rc, "gemm_tcgen05")
        return partials
    rc = lib().ti_gemm_tcgen05(out.data_ptr(), out.stride(0), x.data_ptr(), x.stride(0), w.data_ptr(), n,
                               lin.out_features, k, 1, epilogue, act[0], act[1], act[2], act[3], st.data_ptr(), _stream())
    if rc == 2:
        return None
    check(rc, "gemm_tcgen05")
    return out


MAX_PARTS = 32              # parts of one sequence in decode attention (the combine kernel's limit)


def _align32(n: int) -> int:
    return -(-n // 32) * 32


class SplitKvPlan:
    """How decode attention's B x splits work slots are shared out among the sequences of a step: the
    attention mixer's ``decode_plan``. The tables are computed by C++ (``csrc/host/split_kv_plan.cpp``) while
    the step's metadata is filled; this object carries the native plan to the step planner and tells the
    kernel's caller where the two tables lie in the words the plan was given."""

    def __init__(self, kv_heads: int, page_size: int, pool_tokens: int):
        from . import host
        self._api = host.api()
        self.native = self._api.split_kv_plan_create(kv_heads, page_size, pool_tokens, sm_count(), MAX_PARTS)
        if not self.native:
            raise KernelError(host.last_error())
        self._splits = {}

    def splits(self, batch: int) -> int:
        s = self._splits.get(batch)
        if s is None:
            s = self._splits[batch] = int(self._api.split_kv_plan_splits(self.native, batch))
        return s

    def tables(self, batch: int, words: torch.Tensor):
        """(work [2 * batch * splits], seq [batch]) inside ``words``, the plan's part of the step's metadata."""
        n = 2 * batch * self.splits(batch)
        return words[:n], words[_align32(n):_align32(n) + batch]


def split_tables(lengths, splits: int, page_size: int):
    """The plan's tables for explicit sizes, as numpy arrays work [batch * splits, 2] and seq [batch] (tests and
    micro-benchmarks): work[slot] = (sequence << 16 | part << 8 | parts, or -1: no work; the sequence's length),
    seq[sequence] = first slot << 8 | parts."""
    import ctypes

    import numpy as np
    from . import host
    B = len(lengths)
    work = np.zeros((B * splits, 2), dtype=np.int32)
    seq = np.zeros(B, dtype=np.int32)
    rc = host.api().split_kv_tables(B, splits, page_size, MAX_PARTS, host.longs(int(x) for x in lengths),
                                    work.ctypes.data_as(ctypes.POINTER(ctypes.c_int)), seq.ctypes.data_as(ctypes.POINTER(ctypes.c_int)))
    if rc:
        raise KernelError(host.last_error())
    return work, seq


def decode_splits(batch: int, kv_heads: int, max_context: int) -> int:
    """Split count of decode attention: fixed by the batch size alone, so that a captured step
    stays valid whatever the lengths are (the reference fixes it per model:
    src/ops/tile/attention.jl:250-263)."""
    # Two blocks fit an SM: at most two blocks per SM, so that none has to wait for a second wave.
    want = (2 * sm_count()) // max(1, batch * kv_heads)
    return max(1, min(want, 32, -(-max_context // 64)))


SHORT_PROMPT = 384
SHORT_STEP = 512


def attention(out, q, cache, meta, step, spec) -> bool:
    if q.dtype != torch.bfloat16:
        return False
    if step.is_decode:
        B = step.n_seqs
        # The step's plan carries the split count and how the work slots are shared out among the sequences.
        plan = meta.plan if isinstance(meta.plan, SplitKvPlan) else None
        splits = plan.splits(B) if plan is not None else decode_splits(B, spec.num_kv_heads, cache.k.shape[0] * cache.page_size)
        shared = plan is not None and meta.plan_table is not None and splits > 1
        work, seq = plan.tables(B, meta.plan_table) if shared else (None, None)
        rt_buffer = step.runtime.buffer
        ws_o = rt_buffer("attention.ws_o", (B * splits, spec.num_heads, spec.head_dim), torch.float32)
        ws_ml = rt_buffer("attention.ws_ml", (B * splits, spec.num_heads, 2), torch.float32)
        rc = lib().ti_attention_decode_shared(out.data_ptr(), q.data_ptr(), cache.k.data_ptr(), cache.v.data_ptr(),
                                              meta.block_table.data_ptr(), meta.block_table.stride(0),
                                              step.seq_slots.data_ptr(), step.kv_lens.data_ptr(),
                                              work.data_ptr() if shared else None,
                                              seq.data_ptr() if shared else None, ws_o.data_ptr(),
                                              ws_ml.data_ptr(), spec.scale, B, spec.num_heads, spec.num_kv_heads,
                                              spec.head_dim, cache.page_size, splits, spec.window or 0, _stream())
        if rc == 2:
            return False
        check(rc, "attention_decode")
        if splits > 1:
            add_launches(1)                     # the combine kernel
        return True
    group = spec.num_heads // max(1, spec.num_kv_heads)
    if group < 1 or group > 128 or spec.num_heads % spec.num_kv_heads:
        return False
    tokens_per_tile = 128 // group
    # The tensor-core kernel for the sizes it takes (head size 64 or 128, up to 128 query heads per KV head).
    blocks = sum(-(-n // (2 * tokens_per_tile)) for n in step.host_q_lens)
    # A short step of short sequences (every one ends within SHORT_PROMPT positions, SHORT_STEP tokens in all) takes the
    # mma.sync kernel: with three key steps or fewer per block, and fewer blocks than SMs, the tensor-memory kernel's
    # set-up outweighs its products (a layer of one 256-token prompt: 12 us less; level at 448 tokens; the tensor-memory
    # kernel 2 us ahead at 512, and ahead for four or more prompts of 256 tokens in one step).
    short = step.max_kv_len <= SHORT_PROMPT and step.n_tokens <= SHORT_STEP
    rc = 2 if short else lib().ti_attention_prefill_tc(out.data_ptr(), q.data_ptr(), cache.k.data_ptr(), cache.v.data_ptr(), cache.k.shape[0],
                                       meta.block_table.data_ptr(), meta.block_table.stride(0), step.seq_slots.data_ptr(),
                                       step.cu_seqlens.data_ptr(), step.kv_lens.data_ptr(), step.n_seqs, step.n_tokens, blocks,
                                       spec.scale, spec.num_heads, spec.num_kv_heads, spec.head_dim, cache.page_size,
                                       spec.window or 0, status_word().data_ptr(), _stream())
    if rc != 2:
        check(rc, "attention_prefill_tc")
        return True
    total_tiles = sum(-(-n // tokens_per_tile) for n in step.host_q_lens)
    rc = lib().ti_attention_prefill(out.data_ptr(), q.data_ptr(), cache.k.data_ptr(), cache.v.data_ptr(),
                                    meta.block_table.data_ptr(), meta.block_table.stride(0), step.seq_slots.data_ptr(),
                                    step.cu_seqlens.data_ptr(), step.kv_lens.data_ptr(), step.n_seqs, total_tiles,
                                    spec.scale, spec.num_heads, spec.num_kv_heads, spec.head_dim, cache.page_size,
                                    spec.window or 0, _stream())
    if rc == 2:
        return False
    check(rc, "attention_prefill")
    return True
