"""Host-side choices of the kernels that need no device: the tile width and k slices of the decode-batch
product (``ti_gemm_tcgen05_decode_plan`` in csrc/gemm_tcgen05_decode.cu) and the k slices of the other
decode products. The kernel library is compiled for this (nvcc cross-compiles without a GPU); without
nvcc the test is skipped."""
import ctypes

import pytest

SMS = 148


@pytest.fixture(scope="module")
def plan():
    from tileinfer_b200.kernels import build
    try:
        path = build.build()
    except build.BuildError as e:
        pytest.skip(f"the kernel library cannot be built here: {e}")
    fn = ctypes.CDLL(path).ti_gemm_tcgen05_decode_plan
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_int] * 5 + [ctypes.POINTER(ctypes.c_int)] * 2

    def call(n, out, k, max_splits):
        nt, splits = ctypes.c_int(), ctypes.c_int()
        assert fn(n, out, k, max_splits, SMS, ctypes.byref(nt), ctypes.byref(splits)) == 0
        return nt.value, splits.value
    return call


@pytest.mark.parametrize("n", [9, 33, 64, 100, 128])
@pytest.mark.parametrize("out,k", [(6144, 4096), (4096, 4096), (21504, 4096), (4096, 21504), (131072, 4096), (43008, 8192),
                                   (320, 96), (100, 72), (4099, 264), (16, 8)])
def test_decode_product_plan_is_legal_and_balanced(plan, n, out, k):
    for max_splits in (1, 8):
        nt, splits = plan(n, out, k, max_splits)
        assert nt % 16 == 0 and 16 <= nt <= 256                        # what tcgen05.mma takes as N with 128 rows
        assert 1 <= splits <= max_splits
        k_blocks = -(-k // 64)
        assert splits == 1 or k_blocks // splits >= 8                  # a slice has at least 512 of k
        tiles = -(-out // nt) * splits
        rounds = -(-tiles // SMS)
        # No plan takes more rounds of blocks than the widest tile would, and a last round is never nearly empty
        # when one round less was within reach of a wider tile.
        assert rounds <= -(-(-(-out // 256)) // SMS) + 1
        if max_splits == 1 and out >= 16 * SMS:
            least = -(-out // (256 * SMS))                              # rounds that tiles of 256 rows need
            assert rounds == least, (nt, tiles, rounds, least)


def test_decode_product_plan_at_apertus_8b_sizes(plan):
    """The sizes the cost model was fitted on: one round of blocks for the up projection (135 tiles of 160
    rows, where tiles of 128 need 168 blocks), four for the head."""
    assert plan(64, 21504, 4096, 1) == (160, 1)
    nt, splits = plan(128, 131072, 4096, 1)
    assert splits == 1 and -(-(-(-131072 // nt)) // SMS) == 4
    nt, splits = plan(64, 4096, 21504, 8)
    assert splits > 1 and -(-4096 // nt) * splits <= SMS               # a short, wide product is cut over k into one round


def test_slices_of_the_other_decode_products():
    from tileinfer_b200.kernels import fast
    assert fast.gemv_splits(21504, 4096) == 1 and fast.gemv_splits(4096, 21504) == 1     # 16-row blocks already fill the SMs
    assert fast.gemv_splits(1024, 8192) > 1
    assert fast.tc_splits(21504, 4096, 64) == 1 and fast.tc_splits(4096, 21504, 64) == 8
    assert fast.tc_splits(4096, 4096, 2048) == 1 and fast.tc_splits(4096, 21504, 1024) == 1    # enough tiles for every SM pair: not cut
    # A prompt of a few hundred tokens: products with few output rows have fewer tiles of 256 x 256 than the 74 SM pairs.
    assert fast.tc_splits(4096, 21504, 512) == 2 and fast.tc_splits(4096, 4096, 367) == 2     # 32 tiles -> 64
    assert fast.tc_splits(4096, 21504, 768) == 3                                         # 48 tiles -> 144 in two rounds of a third
    assert fast.tc_splits(4096, 1024, 512) == 1                                          # a slice keeps at least 1,024 of k
    assert fast.tc_splits(8192, 43008, 1024) == 1                                        # 128 tiles, two rounds: four slices would gain 2 %
    assert fast.decode_splits(1, 8, 4096) == 32 and fast.decode_splits(64, 8, 4096) == 1


def test_the_attention_plan_in_the_step_planner_uses_the_same_split_policy():
    """The C++ plan that fills decode attention's work tables and the Python policy that sizes the kernel's
    work space when no plan is attached must agree on the split count for every batch size."""
    from tileinfer_b200.kernels import fast
    for kv_heads, page, pool in ((8, 64, 64 * 4096), (2, 64, 1024), (1, 16, 640), (8, 64, 128)):
        plan = fast.SplitKvPlan(kv_heads, page, pool)
        for batch in (1, 2, 3, 7, 8, 9, 18, 19, 37, 64, 100, 300):
            assert plan.splits(batch) == fast.decode_splits(batch, kv_heads, pool), (kv_heads, pool, batch)
