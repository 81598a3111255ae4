"""The decode-attention entry point that allocates nothing (its work space is an array inside the
library), for hosts that cannot call cudaMalloc: a program whose own pool holds the whole device, or a
loop that must not make a synchronising allocation call. It is called here through its exported C symbol,
twice in a row with different inputs, and must give what the ordinary entry point gives with a work
space allocated by the caller. This file sorts last so that a run stopping at the first failure has
already run every other test; it passes alone in a fresh process as well."""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

SCRATCH_BYTES = 8 << 20


def entry_points():
    from tileinfer_b200.kernels import build
    lib = ctypes.CDLL(build.build())                   # the shared library itself, not the Python wrappers
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.ti_attention_decode_noalloc.restype = I
    lib.ti_attention_decode_noalloc.argtypes = [P, P, P, P, P, I, P, P, F, I, I, I, I, I, I, I, P]
    lib.ti_attention_decode.restype = I
    lib.ti_attention_decode.argtypes = [P, P, P, P, P, I, P, P, P, P, F, I, I, I, I, I, I, I, P]
    lib.ti_last_error.restype = ctypes.c_char_p
    return lib


def case(seed, B, nq, nkv, D, lens):
    g = torch.Generator().manual_seed(seed)
    pages = sum(-(-n // 64) for n in lens) + 2
    k = torch.randn(pages, nkv, 64, D, generator=g).to(torch.bfloat16).cuda()
    v = torch.randn(pages, nkv, 64, D, generator=g).to(torch.bfloat16).cuda()
    q = torch.randn(B, nq, D, generator=g).to(torch.bfloat16).cuda()
    table = torch.zeros(B, max(1, max(-(-n // 64) for n in lens)), dtype=torch.int32)
    order = torch.randperm(pages, generator=g).tolist()
    for b, n in enumerate(lens):
        for i in range(-(-n // 64)):
            table[b, i] = order.pop()
    return q, k, v, table.cuda(), torch.arange(B, dtype=torch.int32).cuda(), torch.tensor(lens, dtype=torch.int32).cuda()


def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row():
    lib = entry_points()
    stream = torch.cuda.current_stream().cuda_stream
    for call, (seed, B, nq, nkv, D, lens, splits) in enumerate([(1, 3, 8, 2, 64, [70, 1, 300], 4), (2, 2, 6, 3, 32, [129, 64], 7)]):
        q, k, v, table, slots, kv_lens = case(seed, B, nq, nkv, D, lens)
        scale = 1 / math.sqrt(D)
        want = torch.full((B, nq, D), float("nan"), dtype=torch.bfloat16, device="cuda")
        ws_o = torch.empty(B, nq, splits, D, device="cuda")
        ws_ml = torch.empty(B, nq, splits, 2, device="cuda")
        rc = lib.ti_attention_decode(want.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), table.data_ptr(), table.stride(0),
                                     slots.data_ptr(), kv_lens.data_ptr(), ws_o.data_ptr(), ws_ml.data_ptr(), scale, B, nq, nkv, D,
                                     64, splits, 0, stream)
        assert rc == 0, lib.ti_last_error()
        got = torch.full((B, nq, D), float("nan"), dtype=torch.bfloat16, device="cuda")
        before = torch.cuda.memory_allocated()
        rc = lib.ti_attention_decode_noalloc(got.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), table.data_ptr(),
                                             table.stride(0), slots.data_ptr(), kv_lens.data_ptr(), scale, B, nq, nkv, D, 64,
                                             splits, 0, stream)
        assert rc == 0, lib.ti_last_error()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert bool(torch.isfinite(got.float()).all()), f"call {call}"
        # Same kernels, same splits: the tests' tolerance for this kernel is a few bfloat16 steps; here the
        # results are in fact identical.
        assert float((got.float() - want.float()).abs().max()) <= 5 * 2.0 ** -8 * float(want.float().abs().max())
        assert torch.equal(got, want)
        # And against exact attention over each sequence's own keys (gathered from its pages), so that the check does
        # not rest on the ordinary entry point alone: softmax(q k / sqrt(D)) v in 64-bit, the new token last.
        for b, n in enumerate(lens):
            pages = table[b, :-(-n // 64)].long()
            keys = k[pages].permute(0, 2, 1, 3).reshape(-1, nkv, D)[:n].double().repeat_interleave(nq // nkv, 1)
            vals = v[pages].permute(0, 2, 1, 3).reshape(-1, nkv, D)[:n].double().repeat_interleave(nq // nkv, 1)
            p = torch.softmax(torch.einsum("hd,khd->hk", q[b].double(), keys) * scale, -1)
            exact = torch.einsum("hk,khd->hd", p, vals)
            assert float((got[b].double() - exact).abs().max()) <= 5 * 2.0 ** -8 * float(exact.abs().max()), (call, b)


def test_a_sequence_without_keys_gives_zeros_not_nan():
    """kv_lens[b] == 0 (an empty request in a batch): zeros, with and without splits, from both entry points' kernels."""
    lib = entry_points()
    stream = torch.cuda.current_stream().cuda_stream
    q, k, v, table, slots, kv_lens = case(5, 2, 4, 2, 64, [0, 70])
    for splits in (1, 3):
        out = torch.full((2, 4, 64), float("nan"), dtype=torch.bfloat16, device="cuda")
        rc = lib.ti_attention_decode_noalloc(out.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), table.data_ptr(), table.stride(0),
                                             slots.data_ptr(), kv_lens.data_ptr(), 0.125, 2, 4, 2, 64, 64, splits, 0, stream)
        assert rc == 0, lib.ti_last_error()
        torch.cuda.synchronize()
        assert float(out[0].float().abs().sum()) == 0.0 and bool(torch.isfinite(out[1].float()).all()) and float(out[1].float().abs().max()) > 0


def test_no_alloc_entry_point_refuses_what_its_array_cannot_hold():
    lib = entry_points()
    q, k, v, table, slots, kv_lens = case(3, 1, 4, 2, 32, [10])
    out = torch.zeros(1, 4, 32, dtype=torch.bfloat16, device="cuda")
    # 4096 sequences x 64 heads x 32 splits x 130 floats is far more than 8 MiB.
    rc = lib.ti_attention_decode_noalloc(out.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), table.data_ptr(), table.stride(0),
                                         slots.data_ptr(), kv_lens.data_ptr(), 0.1, 4096, 64, 8, 128, 64, 32, 0,
                                         torch.cuda.current_stream().cuda_stream)
    assert rc == 1
    text = lib.ti_last_error().decode()
    assert "work space" in text and str(SCRATCH_BYTES) in text
    torch.cuda.synchronize()
    assert float(out.abs().sum()) == 0.0                      # nothing was launched
