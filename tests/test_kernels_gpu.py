"""Each CUDA kernel alone against a plain PyTorch 32-bit reference of the same operation, at sizes
other than the engine's (no powers of two, odd token counts), in float32 and bfloat16."""
import math

import pytest
import torch

import plain_apertus as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def ops():
    from tileinfer_b200.kernels import ops
    return ops


def rnd(x, dtype):
    return x if dtype == torch.float32 else x.to(dtype).float()


def close(got, want, dtype, ulps=2.0, floor=None):
    """Within `ulps` units in the last place of the storage type (the spacing of its numbers at the
    expected value's magnitude), floored at the spacing at the output's RMS: the metric of the
    reference's kernel tests (test/ops/tile.jl:16-20)."""
    got, want = got.float().cpu(), want.float().cpu()
    bits = 23 if dtype == torch.float32 else 7
    floor = floor if floor is not None else float(want.pow(2).mean().sqrt())
    mag = torch.maximum(want.abs(), torch.full_like(want, max(floor, 1e-30)))
    spacing = torch.exp2(torch.floor(torch.log2(mag)) - bits)
    err = ((got - want).abs() / spacing).max()
    assert float(err) <= ulps, f"max error {float(err):.2f} ulps (allowed {ulps})"


def dev(t, dtype=None):
    return (t if dtype is None else t.to(dtype)).cuda().contiguous()


@pytest.mark.parametrize("dtype", DTYPES)
def test_embed_and_gather(ops, dtype):
    torch.manual_seed(0)
    table = dev(torch.randn(301, 100), dtype)
    ids = dev(torch.tensor([0, 300, 7, 7, 150], dtype=torch.int32))
    out = torch.empty(5, 100, dtype=dtype, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.embed(out, table, ids, status)
    assert torch.equal(out, table[ids.long()]) and int(status) == 0
    bad = dev(torch.tensor([3, 301], dtype=torch.int32))
    ops.embed(out[:2], table, bad, status)
    assert int(status) == 2                         # the out-of-range id is reported, not read
    g = torch.empty(3, 100, dtype=dtype, device="cuda")
    ops.gather_rows(g, out, dev(torch.tensor([4, 0, 2], dtype=torch.int32)))
    assert torch.equal(g, out[[4, 0, 2]])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("size", [100, 2560, 4099, 16392])     # the last: longer than the vector kernels' blocks cover
def test_rmsnorm_and_add_rmsnorm(ops, dtype, size):
    torch.manual_seed(1)
    x = rnd(torch.randn(7, size) * 3, dtype)
    w = rnd(1 + 0.2 * torch.randn(size), dtype)
    d = rnd(torch.randn(7, size), dtype)
    want = plain.rmsnorm(x, w, 1e-5, dtype)
    y = torch.empty(7, size, dtype=dtype, device="cuda")
    ops.rmsnorm(y, dev(x, dtype), dev(w, dtype), 1e-5)
    close(y, want, dtype, ulps=1.0 if dtype == torch.bfloat16 else 8.0)
    xs = dev(x, dtype)
    ops.add_rmsnorm(xs, dev(d, dtype), dev(w, dtype), y, 1e-5)
    x2 = rnd(x + d, dtype)
    assert torch.equal(xs.float().cpu(), x2)
    close(y, plain.rmsnorm(x2, w, 1e-5, dtype), dtype, ulps=1.0 if dtype == torch.bfloat16 else 8.0)
    parts = torch.randn(3, 7, size)
    xs = dev(x, dtype)
    ops.add_rmsnorm(xs, None, dev(w, dtype), y, 1e-5, partials=dev(parts))
    x3 = rnd(x + rnd((parts[0] + parts[1]) + parts[2], dtype), dtype)
    assert torch.equal(xs.float().cpu(), x3)


@pytest.mark.parametrize("dtype", DTYPES)
def test_xielu_matches_the_stepwise_formula(ops, dtype):
    torch.manual_seed(2)
    x = rnd(torch.cat([torch.randn(5000) * 4, torch.tensor([0.0, -0.0, -1e-7, 1e-7, -30.0, 30.0])]), dtype)
    for raw in ((18.125, 10.5), (0.3, -0.4)):       # the first layer's large alphas amplify input error
        a = plain.xielu_scalars(torch.tensor(raw[0]), torch.tensor(raw[1]), torch.tensor(0.5), torch.tensor(-1e-6), dtype)
        want = plain.xielu(x, a, dtype)
        y = torch.empty_like(dev(x, dtype))
        ops.xielu(y, dev(x, dtype), float(a.alpha_p), float(a.alpha_n), float(a.beta), float(a.eps))
        if dtype == torch.bfloat16:
            assert torch.equal(y.float().cpu(), want)          # every operation rounds: bit-identical
        else:
            # (expm1(x) - x)·an cancels for small |x|: one unit in the last place of expm1's result, which
            # is what two correct 32-bit expm1 may differ by, is scaled by an. Bound the error by the
            # sizes of the terms that are added, not by the (smaller) result.
            terms = want.abs() + a.alpha_n * (torch.expm1(torch.minimum(x, a.eps)).abs() + x.abs()) + (a.beta * x).abs()
            assert bool(((y.cpu() - want).abs() <= 4 * 2.0 ** -23 * terms).all())


def paged(k, v, page_size, n_pages_total, perm_seed, dtype):
    """Scatter contiguous k, v [len, nkv, D] of several sequences into pools with a shuffled page order.
    Returns pools [pages, nkv, P, D] and the block table rows."""
    g = torch.Generator().manual_seed(perm_seed)
    order = torch.randperm(n_pages_total, generator=g).tolist()
    nkv, D = k[0].shape[1], k[0].shape[2]
    kp = torch.full((n_pages_total, nkv, page_size, D), float("nan"))
    vp = torch.full((n_pages_total, nkv, page_size, D), float("nan"))
    tables = []
    for ks, vs in zip(k, v):
        L = ks.shape[0]
        pages = [order.pop() for _ in range(-(-L // page_size))]
        tables.append(pages)
        pad = len(pages) * page_size - L
        for pool, src in ((kp, ks), (vp, vs)):
            whole = torch.cat([src.float(), torch.full((pad, nkv, D), float("nan"))]) if pad else src.float()
            pool[pages] = whole.view(len(pages), page_size, nkv, D).permute(0, 2, 1, 3)
    kp = torch.nan_to_num(kp, nan=7.0)              # unwritten places hold finite junk, as in a used pool
    vp = torch.nan_to_num(vp, nan=-5.0)
    width = max(len(t) for t in tables) + 2
    table = torch.zeros(len(tables) + 1, width, dtype=torch.int32)
    for i, t in enumerate(tables):
        table[i + 1, :len(t)] = torch.tensor(t)      # slot 0 is left unused on purpose
    return dev(kp, dtype), dev(vp, dtype), dev(table)


def plain_rotation(D, theta, scaling, positions, dtype, rotary=None, interleaved=False):
    """The record the attention-inputs kernel takes, with its table made by the plain implementation
    (32-bit angles, 64-bit cos/sin, rounded to the element type), not by the library's rope part."""
    from types import SimpleNamespace
    rotary = rotary or D
    cfg = plain.read_config({"vocab_size": 8, "hidden_size": 8, "intermediate_size": 8, "num_hidden_layers": 1,
                             "num_attention_heads": 1, "head_dim": rotary, "rms_norm_eps": 1e-5, "rope_theta": theta,
                             "max_position_embeddings": positions, "rope_scaling": scaling})
    cos, sin = plain.rope_tables(cfg, torch.arange(positions), dtype)                   # [positions, rotary], halves equal
    table = torch.stack([cos[:, :rotary // 2], sin[:, :rotary // 2]], -1).contiguous().cuda()
    return SimpleNamespace(cos_sin=table, rotary_dim=rotary, interleaved=interleaved)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,D,n,splits", [(8, 2, 128, 70, 6), (4, 4, 64, 9, 3), (6, 2, 64, 200, 11), (5, 1, 48, 33, 4)])
def test_attention_inputs_from_partial_sums(ops, dtype, nq, nkv, D, n, splits):
    """A projection that was split over k hands its 32-bit partial sums [s, n, features] over; the kernel
    adds them in split order and rounds once, so the result is bit for bit that of the stored projection
    rnd(sum). Head sizes 64 and 128 in bfloat16 take the vector kernel, the rest the general one."""
    torch.manual_seed(11)
    F = (nq + 2 * nkv) * D
    parts = torch.randn(splits, n, F) * torch.logspace(0, -3, splits)[:, None, None]
    total = parts[0].clone()
    for s in range(1, splits):
        total = total + parts[s]                                   # float32, in split order
    stored = rnd(total, dtype)
    rotation = plain_rotation(D, 10000.0, None, 1024, dtype)
    qn, kn = dev(rnd(1 + 0.2 * torch.randn(D), dtype), dtype), dev(rnd(1 + 0.2 * torch.randn(D), dtype), dtype)
    pos = torch.randint(0, 1024, (n,)).int().cuda()
    pages = -(-n // 64) + 1
    smap = torch.randperm(pages * 64)[:n].int().cuda()
    outs = []
    for src in (dev(stored, dtype), dev(parts)):
        q = torch.zeros(n, nq, D, dtype=dtype, device="cuda")
        kp = torch.zeros(pages, nkv, 64, D, dtype=dtype, device="cuda")
        vp = torch.zeros(pages, nkv, 64, D, dtype=dtype, device="cuda")
        ops.attention_inputs(src, q, kp, vp, qn, kn, 1e-5, rotation, pos, smap, nq, nkv, D, 64)
        outs.append((q, kp, vp))
    for a, b in zip(*outs):
        assert torch.equal(a, b)
    assert float(outs[0][0].float().abs().max()) > 0.1 and float(outs[0][2].float().abs().max()) > 0.1


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,D,page", [(6, 3, 32, 64), (5, 1, 48, 16), (8, 2, 128, 64)])
def test_attention_inputs_and_plain_attention(ops, dtype, nq, nkv, D, page):
    """q/k norm + rotation + cache write, then attention over the cache, for two sequences of which one
    continues from cached positions; against the plain whole-sequence functions."""
    torch.manual_seed(3)
    cfg = plain.read_config({"vocab_size": 8, "hidden_size": 8, "intermediate_size": 8, "num_hidden_layers": 1,
                             "num_attention_heads": nq, "num_key_value_heads": nkv, "head_dim": D, "rms_norm_eps": 1e-5,
                             "rope_theta": 10000.0, "max_position_embeddings": 4096,
                             "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "original_max_position_embeddings": 64,
                                              "low_freq_factor": 1.0, "high_freq_factor": 4.0}})
    lens = [150, 77]
    qn, kn = rnd(1 + 0.2 * torch.randn(D), dtype), rnd(1 + 0.2 * torch.randn(D), dtype)
    rotation = plain_rotation(D, 10000.0, {"rope_type": "llama3", "factor": 8.0, "original_max_position_embeddings": 64,
                                           "low_freq_factor": 1.0, "high_freq_factor": 4.0}, 256, dtype)
    qkvs = [rnd(torch.randn(L, (nq + 2 * nkv) * D), dtype) for L in lens]
    n_pages = sum(-(-L // page) for L in lens) + 3
    kp = torch.full((n_pages, nkv, page, D), 3.0, dtype=dtype, device="cuda")
    vp = torch.full((n_pages, nkv, page, D), -2.0, dtype=dtype, device="cuda")
    g = torch.Generator().manual_seed(5)
    order = torch.randperm(n_pages, generator=g).tolist()
    tables = [[order.pop() for _ in range(-(-L // page))] for L in lens]
    table = torch.zeros(3, max(len(t) for t in tables) + 1, dtype=torch.int32)
    for i, t in enumerate(tables):
        table[i + 1, :len(t)] = torch.tensor(t)
    table = table.cuda()
    want_out = []
    for qkv, L in zip(qkvs, lens):
        q = qkv[:, :nq * D].view(L, nq, D); k = qkv[:, nq * D:(nq + nkv) * D].view(L, nkv, D); v = qkv[:, (nq + nkv) * D:].view(L, nkv, D)
        cos, sin = plain.rope_tables(cfg, torch.arange(L), dtype)
        q = plain.rope(plain.rmsnorm(q, qn, 1e-5, dtype), cos, sin, dtype)
        k = plain.rope(plain.rmsnorm(k, kn, 1e-5, dtype), cos, sin, dtype)
        want_out.append(plain.attention(q, k, v, 1 / math.sqrt(D), dtype))
    # Step 1: the first 100 tokens of sequence 0 alone. Step 2: its other 50 together with all of sequence 1.
    def run(entries):
        toks = torch.cat([qkvs[s][a:b] for s, a, b in entries])
        pos = torch.cat([torch.arange(a, b) for s, a, b in entries]).int()
        slot = torch.cat([torch.full((b - a,), s + 1) for s, a, b in entries]).int()
        smap = torch.tensor([tables[s][p // page] * page + p % page for s, a, b in entries for p in range(a, b)]).int()
        n = toks.shape[0]
        q_out = torch.empty(n, nq, D, dtype=dtype, device="cuda")
        ops.attention_inputs(dev(toks, dtype), q_out, kp, vp, dev(qn, dtype), dev(kn, dtype), 1e-5, rotation,
                             pos.cuda(), smap.cuda(), nq, nkv, D, page)
        out = torch.empty(n, nq * D, dtype=dtype, device="cuda")
        ops.attention_plain(out, q_out, kp, vp, table, slot.cuda(), pos.cuda(), 1 / math.sqrt(D), nq, nkv, D, page)
        return out.view(n, nq, D)
    o1 = run([(0, 0, 100)])
    o2 = run([(0, 100, 150), (1, 0, 77)])
    tol = dict(ulps=3.0) if dtype == torch.bfloat16 else dict(ulps=64.0)
    close(o1, want_out[0][:100], dtype, **tol)
    close(o2[:50], want_out[0][100:], dtype, **tol)
    close(o2[50:], want_out[1], dtype, **tol)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D,rotary,interleaved", [(64, 64, True), (64, 32, False), (128, 32, True), (48, 20, True), (32, 32, False)])
def test_attention_inputs_with_a_partial_or_interleaved_rotation(ops, dtype, D, rotary, interleaved):
    """The rotation may cover only the first `rotary` elements of a head and may pair element 2i with 2i + 1
    instead of i with i + rotary/2; written out here with the reference's rounding (each product and the
    sum: src/ops/reference.jl:32-39) and compared exactly."""
    torch.manual_seed(13)
    nq, nkv, n = 3, 2, 45
    rotation = plain_rotation(D, 50000.0, None, 300, dtype, rotary=rotary, interleaved=interleaved)
    qkv = rnd(torch.randn(n, (nq + 2 * nkv) * D), dtype)
    qn, kn = rnd(1 + 0.2 * torch.randn(D), dtype), rnd(1 + 0.2 * torch.randn(D), dtype)
    pos = torch.randint(0, 300, (n,))
    smap = torch.randperm(128)[:n].int()
    q_out = torch.zeros(n, nq, D, dtype=dtype, device="cuda")
    kp = torch.zeros(2, nkv, 64, D, dtype=dtype, device="cuda")
    vp = torch.zeros(2, nkv, 64, D, dtype=dtype, device="cuda")
    ops.attention_inputs(dev(qkv, dtype), q_out, kp, vp, dev(qn, dtype), dev(kn, dtype), 1e-5, rotation, pos.int().cuda(),
                         smap.cuda(), nq, nkv, D, 64)
    table = rotation.cos_sin.cpu()[pos]                                  # [n, rotary/2, 2]
    cos, sin = table[..., 0], table[..., 1]

    def rotate(x):                                                       # x [n, heads, D], already normed
        y = x.clone()
        half = rotary // 2
        for i in range(half):
            a, b = (2 * i, 2 * i + 1) if interleaved else (i, i + half)
            c, s_ = cos[:, i, None], sin[:, i, None]
            y[..., a] = rnd(rnd(x[..., a] * c, dtype) + rnd(-x[..., b] * s_, dtype), dtype)
            y[..., b] = rnd(rnd(x[..., b] * c, dtype) + rnd(x[..., a] * s_, dtype), dtype)
        return y

    q = qkv[:, :nq * D].view(n, nq, D); k = qkv[:, nq * D:(nq + nkv) * D].view(n, nkv, D); v = qkv[:, (nq + nkv) * D:].view(n, nkv, D)
    want_q = rotate(plain.rmsnorm(q, qn, 1e-5, dtype))
    want_k = rotate(plain.rmsnorm(k, kn, 1e-5, dtype))
    lim = dict(ulps=1.0) if dtype == torch.bfloat16 else dict(ulps=16.0)
    close(q_out, want_q, dtype, **lim)
    got_k = kp.view(-1, nkv, 64, D).permute(0, 2, 1, 3).reshape(128, nkv, D)[smap.long()]
    got_v = vp.view(-1, nkv, 64, D).permute(0, 2, 1, 3).reshape(128, nkv, D)[smap.long()]
    close(got_k, want_k, dtype, **lim)
    assert torch.equal(got_v.float().cpu(), v)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,out,k", [(1, 100, 72), (37, 301, 120), (130, 96, 200), (5, 4099, 33), (70, 130, 37), (300, 260, 264),
                                     (64, 40, 1000), (65, 40, 1000)])
def test_gemm_plain_and_epilogues(ops, dtype, n, out, k):
    """The 32-bit product's three kernels (weight streaming up to 64 tokens, 128 x 128 tiles for rows that can be read
    16 bytes at a time, 64 x 64 tiles for the rest) against a 64-bit product, their epilogues, and that a row's
    bits do not depend on which kernel ran or how many rows shared the launch."""
    torch.manual_seed(4)
    x, w = rnd(torch.randn(n, k), dtype), rnd(torch.randn(out, k) * k ** -0.5, dtype)
    want = rnd((x.double() @ w.double().t()).float(), dtype)
    y = torch.empty(n, out, dtype=dtype, device="cuda")
    ops.gemm_plain(y, dev(x, dtype), dev(w, dtype))
    if dtype == torch.bfloat16:
        close(y, want, dtype, ulps=1.0)
    else:
        # The standard bound of a sequential 32-bit sum of k products: k · 2^-24 · sum |x_i w_i|.
        bound = k * 2.0 ** -24 * (x.abs().double() @ w.abs().double().t()).float()
        assert bool(((y.cpu() - want).abs() <= bound).all())
    a = plain.xielu_scalars(torch.tensor(0.3), torch.tensor(-0.4), torch.tensor(0.5), torch.tensor(-1e-6), dtype)
    plain_product = y.clone()
    ops.gemm_plain(y, dev(x, dtype), dev(w, dtype), ops.EPI_XIELU, (float(a.alpha_p), float(a.alpha_n), float(a.beta), float(a.eps)))
    if dtype == torch.bfloat16:
        # The activation is applied to the rounded product: bit-identical on the kernel's own product.
        assert torch.equal(y.float().cpu(), plain.xielu(plain_product.float().cpu(), a, dtype))
    else:
        mine = plain.xielu(plain_product.cpu(), a, dtype)
        assert bool(((y.cpu() - mine).abs() <= 1e-6 * (1 + mine.abs())).all())
    y32 = torch.empty(n, out, dtype=torch.float32, device="cuda")
    ops.gemm_plain(y32, dev(x, dtype), dev(w, dtype), ops.EPI_F32_OUT)
    assert torch.equal(y32.cpu(), plain_product.float().cpu())          # same product, stored in 32-bit
    # A row's result does not depend on how many rows share the launch.
    y1 = torch.empty(1, out, dtype=dtype, device="cuda")
    ops.gemm_plain(y1, dev(x[n - 1:], dtype), dev(w, dtype))
    ops.gemm_plain(y, dev(x, dtype), dev(w, dtype))
    assert torch.equal(y1[0], y[n - 1])


@pytest.mark.parametrize("n", [1, 3, 8, 11, 16])
@pytest.mark.parametrize("out,k", [(100, 72), (301, 120), (4096, 4096), (50, 2000)])
def test_gemv_bf16(ops, n, out, k):
    from tileinfer_b200.kernels.library import check, lib
    torch.manual_seed(5)
    x, w = rnd(torch.randn(n, k), torch.bfloat16), rnd(torch.randn(out, k) * k ** -0.5, torch.bfloat16)
    want = (x.double() @ w.double().t()).float()
    st = torch.cuda.current_stream().cuda_stream
    xd, wd = dev(x, torch.bfloat16), dev(w, torch.bfloat16)
    y = torch.empty(n, out, dtype=torch.bfloat16, device="cuda")
    check(lib().ti_gemv_bf16(y.data_ptr(), out, xd.data_ptr(), k, wd.data_ptr(), n, out, k, 1, 0, 0, 0, 0, 0, st), "gemv")
    close(y, rnd(want, torch.bfloat16), torch.bfloat16, ulps=1.0)
    for splits in (2, 3):
        part = torch.full((splits, n, out), float("nan"), device="cuda")
        check(lib().ti_gemv_bf16(part.data_ptr(), out, xd.data_ptr(), k, wd.data_ptr(), n, out, k, splits, 3, 0, 0, 0, 0, st), "gemv")
        close(part.sum(0), want, torch.float32, ulps=64.0)
    y32 = torch.empty(n, out, dtype=torch.float32, device="cuda")
    check(lib().ti_gemv_bf16(y32.data_ptr(), out, xd.data_ptr(), k, wd.data_ptr(), n, out, k, 1, 2, 0, 0, 0, 0, st), "gemv")
    close(y32, rnd(want, torch.bfloat16), torch.bfloat16, ulps=1.0)
    a = plain.xielu_scalars(torch.tensor(18.125), torch.tensor(10.5), torch.tensor(0.5), torch.tensor(-1e-6), torch.bfloat16)
    check(lib().ti_gemv_bf16(y.data_ptr(), out, xd.data_ptr(), k, wd.data_ptr(), n, out, k, 1, 1, float(a.alpha_p),
                             float(a.alpha_n), float(a.beta), float(a.eps), st), "gemv")
    got, ref = y.float().cpu(), plain.xielu(rnd(want, torch.bfloat16), a, torch.bfloat16)
    # Where the product itself rounds to a neighbouring bfloat16 the activation amplifies it: compare on
    # the kernel's own rounded product instead.
    mine = plain.xielu(y32.cpu(), a, torch.bfloat16)
    assert torch.equal(got, mine)
    close(got, ref, torch.bfloat16, ulps=4.0)


@pytest.mark.parametrize("nq,nkv,D", [(32, 8, 128), (6, 3, 32), (5, 1, 48), (4, 2, 16), (16, 1, 64), (12, 3, 96),
                                      (32, 1, 64), (40, 2, 128), (17, 1, 32)])       # more than 16 query heads per KV head: blocks of 16
def test_attention_decode(ops, nq, nkv, D):
    """Batch of sequences of very different lengths (one key, a page border, hundreds of keys), shuffled
    pages, against exact 32-bit attention. One sequence has a far key made to stand out."""
    from tileinfer_b200.kernels.library import check, lib
    torch.manual_seed(6)
    dtype = torch.bfloat16
    lens = [1, 64, 65, 130, 777, 300]
    B = len(lens)
    ks = [rnd(torch.randn(L, nkv, D), dtype) for L in lens]
    vs = [rnd(torch.randn(L, nkv, D), dtype) for L in lens]
    q = rnd(torch.randn(B, nq, D), dtype)
    # Sequence 4: key 3 (far from the end, in the first page) matches the query of head 0 strongly.
    ks[4][3, 0] = rnd(q[4, 0] * 4.0, dtype)
    n_pages = sum(-(-L // 64) for L in lens) + 4
    kp, vp, table = paged(ks, vs, 64, n_pages, 9, dtype)
    scale = 1 / math.sqrt(D)
    want = torch.stack([plain.attention(q[b:b + 1], ks[b], vs[b], scale, torch.float32, start=lens[b] - 1)[0] for b in range(B)])
    slots = dev(torch.arange(1, B + 1, dtype=torch.int32))
    kv_lens = dev(torch.tensor(lens, dtype=torch.int32))
    st = torch.cuda.current_stream().cuda_stream
    qd = dev(q, dtype)                                  # every device argument stays referenced until the sync
    for splits in (1, 2, 5, 32):
        out = torch.full((B, nq, D), float("nan"), dtype=dtype, device="cuda")
        ws_o = torch.full((B, nq, splits, D), float("nan"), device="cuda")
        ws_ml = torch.full((B, nq, splits, 2), float("nan"), device="cuda")
        check(lib().ti_attention_decode(out.data_ptr(), qd.data_ptr(), kp.data_ptr(), vp.data_ptr(), table.data_ptr(),
                                        table.stride(0), slots.data_ptr(), kv_lens.data_ptr(), ws_o.data_ptr(), ws_ml.data_ptr(),
                                        scale, B, nq, nkv, D, 64, splits, 0, st), "attention_decode")
        close(out, want, dtype, ulps=5.0)
    assert float(want[4, 0].sub(vs[4][3, 0]).abs().max()) < 0.2       # the far key really dominates its head


def test_argmax_ties_go_to_the_smaller_id(ops):
    torch.manual_seed(7)
    logits = torch.randn(5, 1000)
    logits[1, 700] = logits[1, 30] = 9.0
    logits[2] = 0.0                                  # flat
    logits[3, 999] = 50.0                            # all in the last element
    logits[4] = -torch.arange(1000.0)
    out = torch.empty(5, dtype=torch.int32, device="cuda")
    ops.argmax(dev(logits), out)
    assert out.tolist() == [int(logits[0].argmax()), 30, 0, 999, 0]


@pytest.mark.parametrize("V", [1531, 6007])
@pytest.mark.parametrize("temperature,top_k,top_p", [(0.8, 0, 1.0), (1.0, 5, 1.0), (0.7, 50, 0.9), (1.3, 0, 0.5), (1.0, 1, 1.0), (0.5, 200, 0.95)])
def test_device_sampler_follows_the_host_rule(ops, temperature, top_k, top_p, V):
    """Same token as the plain rule for the same (logits, settings, u), except where u × total or top_p
    falls within 1e-5 of a boundary of the cumulative distribution (the reference's own filter,
    test/ops/tile.jl:264-298). In the larger vocabulary the flat row and the row of ties put more tokens
    into one histogram bin than the kernel's fast path gathers, so those rows take its exact path."""
    torch.manual_seed(8)
    rows = 24
    logits = torch.randn(rows, V) * 2.5
    logits[0] = 0.0                                   # flat
    logits[1, 100] = logits[1, 900] = logits[1].max() + 1     # ties at the top
    logits[2, :] = -30.0; logits[2, V - 1] = 5.0             # everything in the last token
    logits[3, ::7] = logits[3, 0]                            # many ties across the k-th
    logits[4, 5:] = logits[4, 5]                             # a few tokens, then one crowd of equals
    seeds = [(1234567 * (r + 1)) & 0xFFFFFFFF for r in range(rows)]
    from tileinfer_b200.sampling.device import _as_i32
    sd = _as_i32(seeds).cuda()
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    checked = 0
    for counter in (0, 1, 17):
        ct = torch.full((rows,), counter, dtype=torch.int32, device="cuda")
        ops.sample(dev(logits), out, temperature, top_k, top_p, sd, ct)
        assert ct.tolist() == [counter + 1] * rows           # the kernel advances the counters
        got = out.tolist()
        for r in range(rows):
            u = plain.sampling_uniform(seeds[r], counter)
            ids, probs = plain.filtered_dist(logits[r], temperature, top_k, top_p)
            cum, near = 0.0, False
            for p in probs:
                cum += p
                if abs(cum - u) < 1e-5:
                    near = True
            if top_p < 1:
                full_ids, full = plain.filtered_dist(logits[r], temperature, top_k, 1.0)
                c = 0.0
                for p in full:
                    c += p
                    if abs(c - top_p) < 1e-5:
                        near = True
            if near:
                continue
            assert got[r] == ids[plain.pick(probs, u)], f"row {r} counter {counter}"
            checked += 1
    assert checked > rows * 2


@pytest.mark.parametrize("V", [131072, 40009, 1531])
@pytest.mark.parametrize("temperature,top_k,top_p", [(0.8, 0, 1.0), (1.0, 40, 0.9), (1.3, 0, 0.5), (0.6, 3, 1.0)])
def test_a_row_shared_by_a_cluster_gives_the_one_block_token(ops, temperature, top_k, top_p, V):
    """The sampler with 2, 4 or 8 blocks per row (their histograms added up and their candidates collected through
    distributed shared memory) chooses what one block per row chooses, on every row: ordinary rows, a flat row and a
    crowd of equals (more tokens in a bin than the fast path gathers: the exact path), everything in the last token,
    ties at the top; and the library's own choice of the sharing agrees with the plain rule away from borders."""
    torch.manual_seed(21)
    rows = 9
    logits = torch.randn(rows, V) * 3.0
    logits[0] = 0.0
    logits[1, 100] = logits[1, V - 7] = logits[1].max() + 1
    logits[2, :] = -30.0; logits[2, V - 1] = 5.0
    logits[3, 5:] = logits[3, 5]
    logits[4, ::3] = logits[4, 0]
    seeds = [(7654321 * (r + 3)) & 0xFFFFFFFF for r in range(rows)]
    from tileinfer_b200.sampling.device import _as_i32
    sd = _as_i32(seeds).cuda()
    lg = dev(logits)
    for counter in (0, 5):
        got = {}
        for share in (1, 2, 4, 8, 0):
            ct = torch.full((rows,), counter, dtype=torch.int32, device="cuda")
            out = torch.full((rows,), -7, dtype=torch.int32, device="cuda")
            ops.sample(lg, out, temperature, top_k, top_p, sd, ct, cluster_blocks=share)
            assert ct.tolist() == [counter + 1] * rows
            got[share] = out.tolist()
        for share in (2, 4, 8, 0):
            assert got[share] == got[1], f"{share} blocks per row, counter {counter}"
        checked = 0
        for r in range(5, rows):                       # the ordinary rows against the plain rule, as in the test above
            u = plain.sampling_uniform(seeds[r], counter)
            ids, probs = plain.filtered_dist(logits[r], temperature, top_k, top_p)
            cum, near = 0.0, False
            for p in probs:
                cum += p
                near = near or abs(cum - u) < 1e-5
            if top_p < 1:
                _, full = plain.filtered_dist(logits[r], temperature, top_k, 1.0)
                c = 0.0
                for p in full:
                    c += p
                    near = near or abs(c - top_p) < 1e-5
            if not near:
                assert got[0][r] == ids[plain.pick(probs, u)], f"row {r} counter {counter}"
                checked += 1
        assert checked >= 2


@pytest.mark.parametrize("nq,nkv,D", [(32, 8, 128), (6, 3, 32), (5, 1, 48), (4, 2, 16), (8, 8, 64), (16, 1, 64)])
def test_attention_prefill(ops, nq, nkv, D):
    """Sequences of unequal lengths in one launch, some continuing from cached positions (start > 0),
    shuffled pages, against exact 32-bit attention. A key far from the queries (hundreds of positions
    back, in the first page) is made to dominate one head, and one sequence is a single token."""
    from tileinfer_b200.kernels.library import check, lib
    torch.manual_seed(11)
    dtype = torch.bfloat16
    total = [300, 1, 130, 513, 64]                  # cached length after the step
    fresh = [300, 1, 30, 200, 64]                   # tokens of the step (the rest was cached before)
    B = len(total)
    ks = [rnd(torch.randn(L, nkv, D), dtype) for L in total]
    vs = [rnd(torch.randn(L, nkv, D), dtype) for L in total]
    qs = [rnd(torch.randn(n, nq, D), dtype) for n in fresh]
    # Sequence 3: key 5 dominates head 1 for its last query (position 512, 507 keys away).
    ks[3][5, 1 // (nq // nkv)] = rnd(qs[3][-1, 1] * 4.0, dtype)
    n_pages = sum(-(-L // 64) for L in total) + 3
    kp, vp, table = paged(ks, vs, 64, n_pages, 13, dtype)
    scale = 1 / math.sqrt(D)
    want = torch.cat([plain.attention(qs[b], ks[b], vs[b], scale, torch.float32, start=total[b] - fresh[b]) for b in range(B)])
    q = dev(torch.cat(qs), dtype)
    cu = [0]
    for n in fresh:
        cu.append(cu[-1] + n)
    tpt = 128 // (nq // nkv)
    tiles = sum(-(-n // tpt) for n in fresh)
    out = torch.full((cu[-1], nq, D), float("nan"), dtype=dtype, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    slots, cu_d, lens_d = (dev(torch.arange(1, B + 1, dtype=torch.int32)), dev(torch.tensor(cu, dtype=torch.int32)),
                           dev(torch.tensor(total, dtype=torch.int32)))
    check(lib().ti_attention_prefill(out.data_ptr(), q.data_ptr(), kp.data_ptr(), vp.data_ptr(), table.data_ptr(), table.stride(0),
                                     slots.data_ptr(), cu_d.data_ptr(), lens_d.data_ptr(), B, tiles, scale, nq, nkv, D, 64, 0, st),
          "attention_prefill")
    close(out, want, dtype, ulps=5.0)
    head = want[cu[4] - 1, 1]
    assert float((head - vs[3][5, 1 // (nq // nkv)]).abs().max()) < 0.2


@pytest.mark.parametrize("nq,nkv,D,window", [(32, 8, 128, 0), (8, 8, 64, 0), (16, 1, 64, 0), (4, 2, 128, 0), (6, 3, 64, 150), (8, 1, 128, 333),
                                             (24, 8, 128, 0), (6, 2, 64, 0), (5, 1, 64, 0), (14, 2, 128, 150), (12, 1, 64, 0),    # groups of 3, 5, 7, 12
                                             (32, 1, 64, 0), (40, 2, 128, 0), (128, 1, 64, 200)])                                  # 32, 20 and 128 heads per KV head
def test_attention_prefill_tensor_core(ops, nq, nkv, D, window):
    """The tcgen05 prefill kernel on unequal sequences in one launch (some continuing from cached
    positions, one a single token, one of several key steps), shuffled pages, with and without a
    window, against exact 32-bit attention. A key hundreds of positions back dominates one head (its
    step raises the row maximum by far more than the lazy rescaling allows to pass), and a key just
    outside a window is made huge and must not show."""
    from tileinfer_b200.kernels import fast
    from tileinfer_b200.kernels.library import check, lib
    torch.manual_seed(17)
    dtype = torch.bfloat16
    total = [700, 1, 130, 513, 64, 257]             # cached length after the step
    fresh = [700, 1, 30, 200, 64, 129]              # tokens of the step (the rest was cached before)
    B, g = len(total), nq // nkv
    ks = [rnd(torch.randn(L, nkv, D), dtype) for L in total]
    vs = [rnd(torch.randn(L, nkv, D), dtype) for L in total]
    qs = [rnd(torch.randn(n, nq, D), dtype) for n in fresh]
    far = 5 if not window else 512 - window + 1     # the farthest key the last query of sequence 3 sees
    ks[3][far, 1 // g] = rnd(qs[3][-1, 1] * 4.0, dtype)
    ks[0][400, 0] = rnd(qs[0][650, 0] * 6.0, dtype)  # found in the fourth key step of a row that began small
    if window:
        ks[3][512 - window, :] = rnd(qs[3][-1, 1] * 9.0, dtype)[None].expand(nkv, D)     # one place outside
    n_pages = sum(-(-L // 64) for L in total) + 3
    kp, vp, table = paged(ks, vs, 64, n_pages, 13, dtype)
    scale = 1 / math.sqrt(D)
    wants = []
    for b in range(B):
        s = torch.einsum("qhd,khd->hqk", qs[b].double(), ks[b].double().repeat_interleave(g, 1)) * scale
        kpos, qpos = torch.arange(total[b]), torch.arange(total[b] - fresh[b], total[b])
        vis = kpos[None, :] <= qpos[:, None]
        if window:
            vis &= kpos[None, :] > qpos[:, None] - window
        pr = s.masked_fill(~vis[None], float("-inf")).softmax(-1)
        wants.append(torch.einsum("hqk,khd->qhd", pr, vs[b].double().repeat_interleave(g, 1)).float())
    want = torch.cat(wants)
    q = dev(torch.cat(qs), dtype)
    cu = [0]
    for n in fresh:
        cu.append(cu[-1] + n)
    per_block = 2 * (128 // g)
    blocks = sum(-(-n // per_block) for n in fresh)
    out = torch.full((cu[-1], nq, D), float("nan"), dtype=dtype, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    slots, cu_d, lens_d = (dev(torch.arange(1, B + 1, dtype=torch.int32)), dev(torch.tensor(cu, dtype=torch.int32)),
                           dev(torch.tensor(total, dtype=torch.int32)))
    status = fast.status_word()
    check(lib().ti_attention_prefill_tc(out.data_ptr(), q.data_ptr(), kp.data_ptr(), vp.data_ptr(), kp.shape[0], table.data_ptr(),
                                        table.stride(0), slots.data_ptr(), cu_d.data_ptr(), lens_d.data_ptr(), B, cu[-1], blocks,
                                        scale, nq, nkv, D, 64, window, status.data_ptr(), st), "attention_prefill_tc")
    fast.check_status()
    close(out, want, dtype, ulps=5.0)
    head = want[cu[4] - 1, 1]
    assert float((head - vs[3][far, 1 // g]).abs().max()) < 0.2


def test_attention_window_edge(ops):
    """With a window of w keys the query at position p sees exactly keys p-w+1 .. p: a key one place
    outside the window is made huge and must not show; plain, prefill and decode kernels agree."""
    from tileinfer_b200.kernels.library import check, lib
    torch.manual_seed(12)
    dtype, nq, nkv, D, L, w = torch.bfloat16, 4, 2, 32, 200, 70
    k = rnd(torch.randn(L, nkv, D), dtype); v = rnd(torch.randn(L, nkv, D), dtype); q = rnd(torch.randn(L, nq, D), dtype)
    k[L - 1 - w] = rnd(q[L - 1, 0] * 8.0, dtype)[None].expand(nkv, D)       # just outside the last query's window
    kp, vp, table = paged([k], [v], 64, 6, 3, dtype)
    scale = 1 / math.sqrt(D)
    s = torch.einsum("qhd,khd->hqk", q, k.repeat_interleave(nq // nkv, 1)) * scale
    pos = torch.arange(L)
    vis = (pos[None, :] <= pos[:, None]) & (pos[None, :] > pos[:, None] - w)
    p = s.masked_fill(~vis[None], float("-inf")).softmax(-1)
    want = torch.einsum("hqk,khd->qhd", p, v.repeat_interleave(nq // nkv, 1))
    st = torch.cuda.current_stream().cuda_stream
    one = dev(torch.ones(1, dtype=torch.int32))
    qd, q_last, cu_d, len_d = dev(q, dtype), dev(q[L - 1:], dtype), dev(torch.tensor([0, L], dtype=torch.int32)), dev(torch.tensor([L], dtype=torch.int32))
    out = torch.empty(L, nq * D, dtype=dtype, device="cuda")
    ops.attention_plain(out, qd, kp, vp, table, dev(torch.ones(L, dtype=torch.int32)), dev(pos.int()), scale, nq, nkv, D, 64, window=w)
    close(out.view(L, nq, D), want, dtype, ulps=4.0)
    out2 = torch.empty(L, nq, D, dtype=dtype, device="cuda")
    check(lib().ti_attention_prefill(out2.data_ptr(), qd.data_ptr(), kp.data_ptr(), vp.data_ptr(), table.data_ptr(), table.stride(0),
                                     one.data_ptr(), cu_d.data_ptr(), len_d.data_ptr(), 1, -(-L // 64), scale, nq, nkv, D, 64, w, st), "prefill")
    close(out2, want, dtype, ulps=5.0)
    out3 = torch.empty(1, nq, D, dtype=dtype, device="cuda")
    ws_o = torch.empty(1, nq, 3, D, device="cuda"); ws_ml = torch.empty(1, nq, 3, 2, device="cuda")
    check(lib().ti_attention_decode(out3.data_ptr(), q_last.data_ptr(), kp.data_ptr(), vp.data_ptr(), table.data_ptr(),
                                    table.stride(0), one.data_ptr(), len_d.data_ptr(),
                                    ws_o.data_ptr(), ws_ml.data_ptr(), scale, 1, nq, nkv, D, 64, 3, w, st), "decode")
    close(out3[0], want[L - 1], dtype, ulps=5.0)


@pytest.mark.parametrize("nq,nkv,D,splits,lengths", [(8, 2, 64, 6, [3, 1500, 64, 129, 700]),
                                                     (40, 2, 64, 5, [7, 1000, 300]),               # 20 query heads per KV head
                                                     (32, 8, 128, 9, [5, 32768, 700, 20000])])    # Apertus-8B heads, long contexts
def test_attention_decode_with_shared_out_slots(ops, nq, nkv, D, splits, lengths):
    """Decode attention over sequences of very unequal lengths with the work slots shared out by length
    (the long sequence read by many blocks, the short ones by one), against exact attention and against
    the same launch with equal splits; up to 32,768 keys, where one sequence gets the most parts there are."""
    import numpy as np
    from tileinfer_b200.kernels.fast import split_tables
    from tileinfer_b200.kernels.library import check, lib
    torch.manual_seed(21)
    dtype = torch.bfloat16
    B, g = len(lengths), nq // nkv
    ks = [rnd(torch.randn(L, nkv, D), dtype) for L in lengths]
    vs = [rnd(torch.randn(L, nkv, D), dtype) for L in lengths]
    qs = rnd(torch.randn(B, nq, D), dtype)
    ks[1][7, 0] = rnd(qs[1, 1] * 4.0, dtype)         # a far key that dominates one head of the long sequence
    kp, vp, table = paged(ks, vs, 64, sum(-(-L // 64) for L in lengths) + 2, 5, dtype)
    scale = 1 / math.sqrt(D)
    want = torch.stack([plain.attention(qs[b:b + 1], ks[b], vs[b], scale, torch.float32, start=lengths[b] - 1)[0] for b in range(B)])
    work, seq = split_tables(np.asarray(lengths, dtype=np.int64), splits, 64)
    assert (seq & 255).tolist()[1] > splits > (seq & 255).tolist()[0]
    st = torch.cuda.current_stream().cuda_stream
    slots, lens_d = dev(torch.arange(1, B + 1, dtype=torch.int32)), dev(torch.tensor(lengths, dtype=torch.int32))
    qd = dev(qs, dtype)
    outs = []
    for tables in ((dev(torch.from_numpy(work).int().reshape(-1)), dev(torch.from_numpy(seq).int())), (None, None)):
        out = torch.full((B, nq, D), float("nan"), dtype=dtype, device="cuda")
        ws_o = torch.full((B * splits, nq, D), float("nan"), device="cuda"); ws_ml = torch.full((B * splits, nq, 2), float("nan"), device="cuda")
        check(lib().ti_attention_decode_shared(out.data_ptr(), qd.data_ptr(), kp.data_ptr(), vp.data_ptr(), table.data_ptr(), table.stride(0),
                                               slots.data_ptr(), lens_d.data_ptr(), tables[0].data_ptr() if tables[0] is not None else None,
                                               tables[1].data_ptr() if tables[1] is not None else None, ws_o.data_ptr(), ws_ml.data_ptr(),
                                               scale, B, nq, nkv, D, 64, splits, 0, st), "decode")
        close(out, want, dtype, ulps=5.0)
        outs.append(out)
    close(outs[0], outs[1].float(), dtype, ulps=2.0)
    assert float((want[1, 1] - vs[1][7, 0]).abs().max()) < 0.2


@pytest.mark.parametrize("n,out,k,splits", [(17, 100, 72, 1), (37, 301, 120, 1), (130, 384, 512, 1), (300, 256, 4160, 1),
                                             (64, 512, 1024, 4), (2048, 256, 192, 1), (40, 4099, 264, 3),
                                             (300, 512, 2048, 2), (700, 777, 4160, 3),      # k slices on SM pairs
                                             (1024, 4900, 8200, 1)])      # the last one takes 256-row blocks
def test_gemm_tcgen05(ops, n, out, k, splits):
    from tileinfer_b200.kernels import fast
    from tileinfer_b200.kernels.library import check, lib
    torch.manual_seed(13)
    dtype = torch.bfloat16
    x, w = rnd(torch.randn(n, k), dtype), rnd(torch.randn(out, k) * k ** -0.5, dtype)
    want = (x.double() @ w.double().t()).float()
    xd, wd = dev(x, dtype), dev(w, dtype)
    st = torch.cuda.current_stream().cuda_stream
    status = fast.status_word()
    def call(y, epi, s=1, act=(0.0, 0.0, 0.0, 0.0)):
        check(lib().ti_gemm_tcgen05(y.data_ptr(), out, xd.data_ptr(), k, wd.data_ptr(), n, out, k, s, epi, *act, status.data_ptr(), st), "tc")
    y = torch.full((n, out), float("nan"), dtype=dtype, device="cuda")
    call(y, 0)
    close(y, rnd(want, dtype), dtype, ulps=1.0)
    y32 = torch.full((n, out), float("nan"), device="cuda")
    call(y32, 2)
    assert torch.equal(y32.cpu(), y.float().cpu())
    a = plain.xielu_scalars(torch.tensor(18.125), torch.tensor(10.5), torch.tensor(0.5), torch.tensor(-1e-6), dtype)
    ya = torch.empty_like(y)
    call(ya, 1, act=(float(a.alpha_p), float(a.alpha_n), float(a.beta), float(a.eps)))
    assert torch.equal(ya.float().cpu(), plain.xielu(y.float().cpu(), a, dtype))
    if splits > 1:
        part = torch.full((splits, n, out), float("nan"), device="cuda")
        call(part, 3, splits)
        close(part.sum(0), want, torch.float32, ulps=64.0)
    fast.check_status()


@pytest.mark.parametrize("n,out,k,tile,splits", [(9, 100, 72, 16, 1), (37, 301, 120, 48, 1), (64, 512, 1024, 112, 4), (128, 384, 512, 256, 1),
                                                 (100, 4099, 264, 160, 3), (17, 2000, 4160, 240, 2), (64, 1000, 584, 0, 1),
                                                 (130, 301, 120, 48, 1), (200, 1000, 584, 0, 1), (256, 700, 2048, 112, 2),     # two halves of 128 tokens
                                                 (255, 512, 1024, 256, 1),
                                                 (33, 3000, 200, 32, 1)])     # the last one: a block walks several tiles
def test_gemm_tcgen05_decode(ops, n, out, k, tile, splits):
    """The decode-batch product (tokens in the tensor-memory lanes, weight rows in tiles of any multiple of 16)
    against a 64-bit product: every epilogue, ragged last tiles, k that is no multiple of 64, k slices."""
    from tileinfer_b200.kernels import fast
    from tileinfer_b200.kernels.library import check, lib
    torch.manual_seed(17)
    dtype = torch.bfloat16
    x, w = rnd(torch.randn(n, k), dtype), rnd(torch.randn(out, k) * k ** -0.5, dtype)
    want = (x.double() @ w.double().t()).float()
    xd, wd = dev(x, dtype), dev(w, dtype)
    st = torch.cuda.current_stream().cuda_stream
    status = fast.status_word()
    def call(y, epi, s=1, act=(0.0, 0.0, 0.0, 0.0)):
        check(lib().ti_gemm_tcgen05_decode(y.data_ptr(), out, xd.data_ptr(), k, wd.data_ptr(), n, out, k, tile, s, epi, *act,
                                           status.data_ptr(), st), "tc decode")
    y = torch.full((n, out), float("nan"), dtype=dtype, device="cuda")
    call(y, 0)
    close(y, rnd(want, dtype), dtype, ulps=1.0)
    y32 = torch.full((n, out), float("nan"), device="cuda")
    call(y32, 2)
    assert torch.equal(y32.cpu(), y.float().cpu())
    a = plain.xielu_scalars(torch.tensor(18.125), torch.tensor(10.5), torch.tensor(0.5), torch.tensor(-1e-6), dtype)
    ya = torch.empty_like(y)
    call(ya, 1, act=(float(a.alpha_p), float(a.alpha_n), float(a.beta), float(a.eps)))
    assert torch.equal(ya.float().cpu(), plain.xielu(y.float().cpu(), a, dtype))
    if splits > 1:
        part = torch.full((splits, n, out), float("nan"), device="cuda")
        call(part, 3, splits)
        # 32-bit sums of k products of bfloat16 numbers: the rounding error grows like the square root of k.
        close(part.sum(0), want, torch.float32, ulps=4.0 * k ** 0.5)
        close(rnd(part.sum(0).cpu(), dtype), rnd(want, dtype), dtype, ulps=1.0)
    # Rows past the last token and features past the last row are never written.
    guard = torch.full((n + 3, out + 5), 7.0, dtype=dtype, device="cuda")
    check(lib().ti_gemm_tcgen05_decode(guard.data_ptr(), out + 5, xd.data_ptr(), k, wd.data_ptr(), n, out, k, tile, 1, 0, 0.0, 0.0, 0.0, 0.0,
                                       status.data_ptr(), st), "tc decode")
    assert torch.equal(guard[:n, :out].float().cpu(), y.float().cpu())
    assert bool((guard[n:] == 7.0).all()) and bool((guard[:, out:] == 7.0).all())
    fast.check_status()


@pytest.mark.parametrize("raw", [(18.125, 10.5), (0.3, -0.4)])
def test_xielu_over_every_bfloat16_value(ops, raw):
    """The activation has 65,280 possible finite inputs in bfloat16: every one of them through the element-wise
    kernel and through the epilogue of every product kernel (the products have one-hot weight rows, so that
    the sums ARE the inputs), bit for bit against the step-wise formula. An approximation of expm1 that rounds
    one input differently shows here."""
    from tileinfer_b200.kernels import fast
    from tileinfer_b200.kernels.library import check, lib
    dtype = torch.bfloat16
    bits = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(torch.bfloat16)
    vals = bits[torch.isfinite(bits.float())]
    assert vals.numel() == 65280
    a = plain.xielu_scalars(torch.tensor(raw[0]), torch.tensor(raw[1]), torch.tensor(0.5), torch.tensor(-1e-6), dtype)
    act = (float(a.alpha_p), float(a.alpha_n), float(a.beta), float(a.eps))
    want = plain.xielu(vals.float(), a, dtype)
    y = torch.empty(vals.numel(), dtype=dtype, device="cuda")
    ops.xielu(y, vals.cuda(), *act)
    assert torch.equal(y.float().cpu(), want)
    # As products: x [1020 tokens, 64] holds the values, W [128, 64] has row j = unit vector j mod 64.
    k, out = 64, 128
    x = vals.view(-1, k)
    w = torch.zeros(out, k)
    w[torch.arange(out), torch.arange(out) % k] = 1.0
    wd = dev(w, dtype)
    want2 = want.view(-1, k).repeat(1, 2)
    st = torch.cuda.current_stream().cuda_stream
    status = fast.status_word()
    for lo, hi in ((0, 1020), (0, 128), (128, 192), (192, 200)):      # 1,020 tokens at once, then steps of 128, 64 and 8
        xd = x[lo:hi].contiguous().cuda()
        n = hi - lo
        got = {}
        y2 = torch.full((n, out), float("nan"), dtype=dtype, device="cuda")
        check(lib().ti_gemm_tcgen05(y2.data_ptr(), out, xd.data_ptr(), k, wd.data_ptr(), n, out, k, 1, 1, *act, status.data_ptr(), st), "tc")
        got["tcgen05"] = y2
        if n <= 128:
            y3 = torch.full((n, out), float("nan"), dtype=dtype, device="cuda")
            check(lib().ti_gemm_tcgen05_decode(y3.data_ptr(), out, xd.data_ptr(), k, wd.data_ptr(), n, out, k, 0, 1, 1, *act,
                                               status.data_ptr(), st), "tc decode")
            got["tcgen05 decode"] = y3
        if n <= 16:
            y4 = torch.full((n, out), float("nan"), dtype=dtype, device="cuda")
            check(lib().ti_gemv_bf16(y4.data_ptr(), out, xd.data_ptr(), k, wd.data_ptr(), n, out, k, 1, 1, *act, st), "gemv")
            got["weight streaming"] = y4
        y5 = torch.full((n, out), float("nan"), dtype=dtype, device="cuda")
        ops.gemm_plain(y5, xd, wd, ops.EPI_XIELU, act)
        got["plain"] = y5
        for name, yy in got.items():
            assert torch.equal(yy.float().cpu(), want2[lo:hi]), f"{name}, tokens {lo} to {hi}"
    fast.check_status()


def test_a_wait_that_runs_out_is_reported_and_the_device_goes_on(ops):
    """The error path of the bounded waits: a barrier that nothing completes, waited on with a limit of
    1,024 attempts. The kernel returns, the wait's bit is in the status word, check_status() raises and
    clears it, and the next tensor-core product runs clean."""
    from tileinfer_b200.kernels import fast
    from tileinfer_b200.kernels.library import KernelError, check, lib
    fast.check_status()
    status = fast.status_word()
    result = torch.zeros(1, dtype=torch.int32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    check(lib().ti_wait_probe(status.data_ptr(), 7, 1024, result.data_ptr(), st), "wait_probe")
    torch.cuda.synchronize()
    assert int(result.item()) == 2 and int(status.item()) == 1 << 7
    with pytest.raises(KernelError, match=r"gave up waiting.*\[7\]"):
        fast.check_status()
    assert int(status.item()) == 0
    torch.manual_seed(1)
    x, w = rnd(torch.randn(40, 256), torch.bfloat16), rnd(torch.randn(128, 256) / 16, torch.bfloat16)
    y = torch.empty(40, 128, dtype=torch.bfloat16, device="cuda")
    xd, wd = dev(x, torch.bfloat16), dev(w, torch.bfloat16)
    rc = lib().ti_gemm_tcgen05(y.data_ptr(), 128, xd.data_ptr(), 256, wd.data_ptr(), 40, 128, 256, 1, 0, 0.0, 0.0, 0.0, 0.0,
                               status.data_ptr(), st)
    assert rc == 0
    close(y, rnd((x.double() @ w.double().t()).float(), torch.bfloat16), torch.bfloat16, ulps=1.0)
    fast.check_status()


def test_new_pages_reach_the_device_table_and_their_values_are_zeroed(ops):
    """The cache's books (C++) write a fresh page's block-table entry to the device and zero its VALUES in every
    layer of the group with one kernel; keys and pages that were not taken are left alone. Many pages at once
    (more than one launch's worth of writes), two groups, slots given back and taken again."""
    from tileinfer_b200.cache import Cache
    from tileinfer_b200.parts import CacheRequest
    reqs = [CacheRequest("paged_kv", kv_heads=2, head_dim=16), CacheRequest("paged_kv", kv_heads=2, head_dim=16),
            CacheRequest("paged_kv", kv_heads=1, head_dim=48), CacheRequest("paged_kv", kv_heads=2, head_dim=16)]
    cache = Cache(reqs, torch.bfloat16, "cuda", max_tokens=64 * 200, max_seqs=4, page_size=64)
    assert [g.layers for g in cache.paged_groups] == [[0, 1, 3], [2]]
    for g in cache.paged_groups:
        g.k.fill_(float("nan")); g.v.fill_(float("nan"))
    a, b = cache.alloc_slot(), cache.alloc_slot()
    cache.reserve([(a, 64 * 150 + 1), (b, 70)])                 # 151 + 2 pages: three launches of writes per group
    torch.cuda.synchronize()
    for g in cache.paged_groups:
        assert torch.equal(g.device_table.cpu(), g.host_table)
        taken = torch.tensor(sorted(p for t in g.tables.values() for p in t))
        assert len(taken) == 153 and g.pages.held == 153
        free = torch.tensor([p for p in range(g.num_pages) if not g.pages.is_held(p)])
        assert float(g.v[:, taken].float().abs().sum()) == 0.0                      # zeroed in every layer of the group
        assert bool(torch.isnan(g.v[:, free].float()).all()) and bool(torch.isnan(g.k.float()).all())
    cache.advance(a, 64 * 150 + 1); cache.advance(b, 70)
    cache.free_slot(a)
    for g in cache.paged_groups:
        g.v.fill_(float("nan"))
    c = cache.alloc_slot()
    assert c == a
    cache.reserve([(c, 65)])                                    # the lowest free pages again: they were a's
    torch.cuda.synchronize()
    for g in cache.paged_groups:
        pages = torch.tensor(g.tables[c])
        assert g.tables[c] == [0, 1] and torch.equal(g.device_table[c, :2].cpu(), pages.int())
        assert float(g.v[:, pages].float().abs().sum()) == 0.0 and bool(torch.isnan(g.v[:, torch.tensor(g.tables[b])].float()).all())
