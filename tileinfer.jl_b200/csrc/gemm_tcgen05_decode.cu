// Tensor-core product for decode batches and short prompts (up to 256 tokens): y[n, out] = x[n, in] · W[out, in]ᵀ in
// bfloat16 with 32-bit accumulation, built to stream W once from HBM with every SM equally loaded.
//
// Here the TOKENS are the 128-row operand of tcgen05.mma (rows beyond n are zero-filled by TMA and
// their results never read) and the WEIGHT rows are the N operand, whose width may be any multiple of
// 16 up to 256. So the rows of W can be cut into as many tiles as there are SMs, whatever `out` is
// (21,504 rows: 135 tiles of 160; 131,072 rows: 586 tiles of 224 = 3.96 rounds of 148), where tiles of
// a fixed 128 rows leave either a ragged second round or SMs with a short pipeline. One block per SM
// owns all of the SM's shared memory: a stage holds 64 of k (16 KB of tokens, 128 bytes per weight
// row), five to eight stages deep, which keeps 100 to 160 KB of weight loads in flight per SM. A step of
// 129 to 256 tokens is two such token tiles per stage and two accumulators: the weights are still read once.
// Products with few rows are also cut over k (32-bit partial sums [split, n, out], added in split
// order by the consumer), with fewer and longer slices than tiles of 128 rows need.
//
// Warp 0 produces (TMA), warp 1 issues the MMAs, warps 2-17 run the epilogue: a thread owns one token
// (its tensor-memory lane) and writes 32 consecutive features at a time, 64 or 128 contiguous bytes.
// Epilogues: round to bfloat16; xIELU on the rounded sums; 32-bit logits; raw partial sums.
// Every wait on an mbarrier is bounded (tcgen05.cuh).
//
// AntoineBut/TileInfer.jl has no counterpart: it runs one sequence, so its decode product is a GEMV
// (src/ops/tile/linear.jl:15-29); the roundings are those of its GEMM (linear.jl:80-100).
#include "tcgen05.cuh"
#include "tensor_map.h"

namespace {

using namespace tc;

constexpr int BMT = 128;           // token rows of the MMA (tensor-memory lanes)
constexpr int BK = 64;             // k per stage: one 128-byte swizzle row
constexpr int A_BYTES = BMT * BK * 2;
constexpr int MAX_STAGES = 8;
constexpr int EPI_WARPS = 16;          // four per quarter of the tensor-memory lanes: with 64 tokens or fewer only two quarters have work
constexpr int THREADS = 64 + 32 * EPI_WARPS;
constexpr int SMEM_LIMIT = 227 * 1024;
constexpr int SM_COUNT_DEFAULT = 148;

enum { EPI_NONE = 0, EPI_XIELU = 1, EPI_F32 = 2, EPI_PARTIAL = 3 };

struct Params {
    int M, N, K;                   // out features, tokens, in features
    int nt;                        // weight rows per tile (multiple of 16, at most 256)
    int m_tiles, splits, k_blocks;
    int stages, stage_bytes, tmem_cols;
    int rotate;                    // every weight tile starts at another place of its k range
    int halves, acc_stride;        // 128-token halves of the step (1 or 2) and the tensor-memory columns between their accumulators
    long long ldy;
    int epilogue;
    XieluParams act;
    int* status;
};

struct TileIter {
    int id, step, total;
    int m, split, kb_lo, kb_hi, rot;
    __device__ bool next(const Params& p) {
        if (id >= total) return false;
        split = id % p.splits;
        m = id / p.splits;
        kb_lo = (int)((long long)p.k_blocks * split / p.splits);
        kb_hi = (int)((long long)p.k_blocks * (split + 1) / p.splits);
        rot = p.rotate ? (m * 7) % (kb_hi - kb_lo) : 0;
        id += step;
        return true;
    }
    __device__ int kb_at(int i) const { const int n_kb = kb_hi - kb_lo; int k = i + rot; if (k >= n_kb) k -= n_kb; return kb_lo + k; }
};

// The stores of one thread's chunk: `count` consecutive features of one token, starting at a multiple of 16.
__device__ __forceinline__ void store_bf16_chunk(bf16* dst, const unsigned* o, int count, int m, int M, bool vec) {
    if (vec && m + count <= M) {
#pragma unroll
        for (int j = 0; j < 32; j += 8)
            if (j < count)
                *reinterpret_cast<uint4*>(dst + j) = make_uint4(o[j] | (o[j + 1] << 16), o[j + 2] | (o[j + 3] << 16),
                                                                o[j + 4] | (o[j + 5] << 16), o[j + 6] | (o[j + 7] << 16));
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (j < count && m + j < M) reinterpret_cast<unsigned short*>(dst)[j] = (unsigned short)o[j];
    }
}
__device__ __forceinline__ void store_f32_chunk(float* dst, const float* v, int count, int m, int M, bool vec) {
    if (vec && m + count <= M) {
#pragma unroll
        for (int j = 0; j < 32; j += 4)
            if (j < count) *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (j < count && m + j < M) dst[j] = v[j];
    }
}

__device__ __forceinline__ unsigned instr_desc_rt(int n) {
    // kind::f16: D 32-bit, A and B bfloat16, both K-major, M = 128, N = n.
    return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(BMT >> 4) << 24);
}

__global__ void __launch_bounds__(THREADS, 1) gemm_tcgen05_decode_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                         const __grid_constant__ CUtensorMap map_x,
                                                                         void* __restrict__ y, Params p) {
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);   // swizzled tiles: 1024-byte alignment
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(tiles + (size_t)p.stages * p.stage_bytes);
    // bars: full[MAX_STAGES], empty[MAX_STAGES], acc_full, acc_empty; then the tensor-memory base address.
    const unsigned full0 = smem_addr(bars), empty0 = full0 + 8 * MAX_STAGES;
    const unsigned accf = empty0 + 8 * MAX_STAGES, acce = accf + 8;
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 2 * MAX_STAGES + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        mbar_init(accf, 1);
        mbar_init(acce, EPI_WARPS);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_addr(tmem_slot), (unsigned)p.tmem_cols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    TileIter it;
    it.id = blockIdx.x; it.step = gridDim.x; it.total = p.m_tiles * p.splits;
    const int b_bytes = p.nt * BK * 2, a_bytes = p.halves * A_BYTES;

    // The weights do not depend on the previous kernel: the loads of the first tile's first weight blocks
    // (as many as there are stages) are on their way before the wait for it. Its results (the tokens,
    // and the output buffer it may still read) are touched only afterwards.
    int ahead = 0;
    if (warp == 0) {
        TileIter first = it;
        if (first.next(p)) {
            ahead = min(p.stages, first.kb_hi - first.kb_lo);
            if (lane == 0)
                for (int s = 0; s < ahead; ++s) {
                    const unsigned bar = full0 + 8 * s;
                    mbar_expect_tx(bar, (unsigned)(a_bytes + b_bytes));
                    tma_load_2d(smem_addr(tiles + (size_t)s * p.stage_bytes) + a_bytes, &map_w, first.kb_at(s) * BK, first.m * p.nt, bar);
                }
            __syncwarp();
        }
    }
    pdl_wait();
    pdl_launch_dependents();
    const unsigned tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------------------------------------------------------- producer (TMA), one thread
        int stage = 0, issued = 0;
        unsigned phase = 0;
        bool ok = true;
        while (lane == 0 && ok && it.next(p)) {
            for (int i = 0; i < it.kb_hi - it.kb_lo; ++i, ++issued) {
                const int kb = it.kb_at(i);
                ok = mbar_wait(empty0 + 8 * stage, phase ^ 1, p.status, 11);
                if (!ok) break;
                const unsigned bar = full0 + 8 * stage;
                const unsigned dst = smem_addr(tiles + (size_t)stage * p.stage_bytes);
                if (issued >= ahead) {                      // else this stage's weights are already on their way
                    mbar_expect_tx(bar, (unsigned)(a_bytes + b_bytes));
                    tma_load_2d(dst + a_bytes, &map_w, kb * BK, it.m * p.nt, bar);
                }
                for (int h = 0; h < p.halves; ++h) tma_load_2d(dst + h * A_BYTES, &map_x, kb * BK, h * BMT, bar);
                if (++stage == p.stages) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer, one thread
        int stage = 0, local = 0;
        unsigned phase = 0;
        bool ok = true;
        const unsigned idesc = instr_desc_rt(p.nt);
        while (lane == 0 && ok && it.next(p)) {
            ok = mbar_wait(acce, (unsigned)((local & 1) ^ 1), p.status, 12);   // the epilogue has read the last tile
            if (!ok) break;
            tc_fence_after();
            for (int i = 0; i < it.kb_hi - it.kb_lo; ++i) {
                ok = mbar_wait(full0 + 8 * stage, phase, p.status, 13);
                if (!ok) break;
                tc_fence_after();
                const unsigned a_addr = smem_addr(tiles + (size_t)stage * p.stage_bytes);
                const unsigned long long db = smem_desc_sw128(a_addr + a_bytes);
                for (int h = 0; h < p.halves; ++h) {       // the second 128 tokens of a step of up to 256 have an accumulator of their own
                    const unsigned long long da = smem_desc_sw128(a_addr + h * A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)      // 16 of k = 32 bytes further along the swizzled row
                        umma_bf16(tmem_base + (unsigned)(h * p.acc_stride), da + (unsigned long long)(2 * k), db + (unsigned long long)(2 * k), idesc,
                                  (i > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(empty0 + 8 * stage);           // the stage is free once these MMAs have read it
                if (++stage == p.stages) { stage = 0; phase ^= 1; }
            }
            if (!ok) break;
            umma_commit(accf);                             // the accumulator is complete
            ++local;
        }
    } else {
        // ---------------------------------------------------------------- epilogue (16 warps)
        const int quarter = warp & 3;                      // the tensor-memory lanes this warp may read
        const int col_group = (warp - 2) >> 2;             // four warps share a quarter: chunks of 32 columns go round among them
        const bool vec_bf16 = (p.ldy % 8 == 0) && (((uintptr_t)y & 15) == 0);
        const bool vec_f32 = (p.ldy % 4 == 0) && (((uintptr_t)y & 15) == 0);
        const XieluPacked act = xielu_pack(p.act);
        int local = 0;
        bool ok = true;
        while (ok && it.next(p)) {
            ok = __all_sync(0xffffffffu, mbar_wait(accf, (unsigned)(local & 1), p.status, 14));
            if (!ok) break;
            tc_fence_after();
            const int m0 = it.m * p.nt;
            const int cols = min(p.nt, p.M - m0);          // features of this tile that exist
            for (int h = 0; h < p.halves; ++h) {
            const int token = h * BMT + quarter * 32 + lane;
            if (h * BMT + quarter * 32 < p.N) {            // uniform across the warp: some of its tokens exist
                const unsigned t_row = tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(h * p.acc_stride);
#pragma unroll 1
                for (int c = col_group * 32; c < cols; c += (EPI_WARPS / 4) * 32) {
                    const int count = min(32, p.nt - c);   // 32, or 16 at the end of a tile whose width is an odd multiple of 16
                    unsigned r[32];
                    if (count == 32) tmem_ld32(t_row + c, r); else tmem_ld16(t_row + c, r);
                    tmem_ld_wait();
                    const int m = m0 + c;
                    if (p.epilogue >= EPI_F32) {
                        float v[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const float s = __uint_as_float(r[j]);
                            v[j] = p.epilogue == EPI_PARTIAL ? s : rnd<bf16>(s);
                        }
                        if (token < p.N) {
                            float* dst = (float*)y + ((size_t)(p.epilogue == EPI_PARTIAL ? it.split : 0) * p.N + token) * p.ldy + m;
                            store_f32_chunk(dst, v, count, m, p.M, vec_f32);
                        }
                    } else {
                        unsigned o[32];                    // bfloat16 bits in the low halves
#pragma unroll
                        for (int j = 0; j < 32; j += 2) {
                            const float s0 = __uint_as_float(r[j]), s1 = __uint_as_float(r[j + 1]);
                            if (p.epilogue == EPI_XIELU) {
                                xielu_bf16_pair(s0, s1, act, o[j], o[j + 1]);
                            } else {
                                const __nv_bfloat162 q = __floats2bfloat162_rn(s0, s1);
                                const unsigned bits = *reinterpret_cast<const unsigned*>(&q);
                                o[j] = bits & 0xffffu; o[j + 1] = bits >> 16;
                            }
                        }
                        if (token < p.N) store_bf16_chunk((bf16*)y + (size_t)token * p.ldy + m, o, count, m, p.M, vec_bf16);
                    }
                }
            }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acce);
            ++local;
        }
    }
    if (*reinterpret_cast<volatile int*>(p.status) != 0) drain_after_timeout();   // a wait ran out somewhere: let what is in flight land
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, (unsigned)p.tmem_cols);
    }
}

int tensor_map_2d(CUtensorMap* out, const void* ptr, unsigned long long rows, unsigned long long cols, unsigned long long ld,
                  unsigned box_rows) {
    const unsigned long long dims[2] = {cols, rows};
    const unsigned long long strides[1] = {ld * 2};
    const unsigned box[2] = {(unsigned)BK, box_rows};
    return ti_tensor_map_bf16(out, ptr, 2, dims, strides, box, true);
}

int stages_for(int nt, int halves = 1) {
    const int stage = halves * A_BYTES + nt * BK * 2;
    const int fit = (SMEM_LIMIT - 1024 /*alignment*/ - 256 /*barriers*/) / stage;
    return fit > MAX_STAGES ? MAX_STAGES : fit;
}

// The tile width and the number of k slices for a product: the pair with the shortest estimated time.
// The estimate is fitted to measurements on Apertus-8B products (16 to 128 tokens, every width, 1 to 8
// slices): a block takes 0.38 us + 1.25 ns per weight row for each 64 of k, whatever the token count; the
// device streams at most about 5.2 TB/s in this pattern; a tile costs about 2 us beyond its k loop; and
// the consumer adds the partial sums of k slices at about 0.9 TB/s (one block per token).
void plan(int n, int out, int in, int max_splits, int sm_count, int* nt_out, int* splits_out) {
    const int k_blocks = (in + BK - 1) / BK;
    const double kb_us = 0.38, row_us = 0.00125, hbm_per_us = 5.2e6, tile_us = 2.0, partial_per_us = 0.9e6;
    const double floor_us = (double)out * (double)in * 2.0 / hbm_per_us;
    double best = 1e30;
    int best_nt = 128, best_s = 1;
    for (int s = 1; s <= max_splits && s <= 8; ++s) {
        if (s > 1 && k_blocks / s < 8) break;              // a slice has at least 512 of k
        for (int nt = 16; nt <= 256; nt += 16) {
            if (stages_for(nt, n > BMT ? 2 : 1) < 3) continue;
            const long long tiles = (long long)((out + nt - 1) / nt) * s;
            const long long rounds = (tiles + sm_count - 1) / sm_count;
            const double kb = (double)((k_blocks + s - 1) / s);
            double t = (double)rounds * (kb * (kb_us + row_us * nt) + tile_us);
            if (t < floor_us) t = floor_us;
            if (s > 1) t += (double)(s - 1) * (double)n * (double)out * 4.0 / partial_per_us;
            if (t < best) { best = t; best_nt = nt; best_s = s; }
        }
    }
    *nt_out = best_nt;
    *splits_out = best_s;
}

int device_sm_count() {
    static int sm_count = 0;
    if (!sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (sm_count <= 0) sm_count = SM_COUNT_DEFAULT;
    }
    return sm_count;
}

}  // namespace

// The tile width (`nt`) and number of k slices (`splits`, at most `max_splits`) this file would choose
// for a product of `n` tokens; `sm_count` 0 asks the current device. Needs no GPU when sm_count is given.
extern "C" int ti_gemm_tcgen05_decode_plan(int n, int out, int in, int max_splits, int sm_count, int* nt, int* splits) {
    TI_REQUIRE(n >= 1 && out >= 1 && in >= 1 && nt != nullptr && splits != nullptr, "gemm_tcgen05_decode_plan: bad arguments");
    plan(n, out, in, max_splits < 1 ? 1 : max_splits, sm_count > 0 ? sm_count : device_sm_count(), nt, splits);
    return 0;
}

// y: [n, ldy] bfloat16 (float32 for the logits epilogue), or partial sums [splits, n, ldy] float32 for the
// partial epilogue. n <= 256 (from 129 tokens on as two halves of 128 with an accumulator each). `nt` and `splits` as given by the plan (nt 0: plan here, with no k slices).
// `status` is a device word that must be zero; non-zero afterwards means a wait ran out.
// Returns 2 when the sizes are outside what the kernel takes (the caller then uses another product).
extern "C" int ti_gemm_tcgen05_decode(void* y, long long ldy, const void* x, long long ldx, const void* W, int n, int out, int in,
                                      int nt, int splits, int epilogue, float alpha_p, float alpha_n, float beta, float eps,
                                      int* status, cudaStream_t stream) {
    if (n == 0) return 0;
    if (n > 2 * BMT || in % 8 != 0 || ldx % 8 != 0 || ((uintptr_t)W & 15) || ((uintptr_t)x & 15) || in < 8) {
        ti_fail("gemm_tcgen05_decode takes up to %d tokens and 16-byte aligned rows: n=%d, in=%d, ldx=%lld", 2 * BMT, n, in, ldx);
        return 2;
    }
    TI_REQUIRE(epilogue >= 0 && epilogue <= 3, "gemm_tcgen05_decode: unknown epilogue %d", epilogue);
    TI_REQUIRE(status != nullptr, "gemm_tcgen05_decode: status word missing");
    const int sm_count = device_sm_count();
    if (nt <= 0) plan(n, out, in, 1, sm_count, &nt, &splits);
    TI_REQUIRE(nt % 16 == 0 && nt >= 16 && nt <= 256, "gemm_tcgen05_decode: tile width %d (a multiple of 16 up to 256)", nt);
    Params p;
    p.M = out; p.N = n; p.K = in; p.nt = nt;
    p.m_tiles = (out + nt - 1) / nt;
    p.k_blocks = (in + BK - 1) / BK;
    p.splits = splits < 1 ? 1 : (splits > p.k_blocks ? p.k_blocks : splits);
    TI_REQUIRE(p.splits == splits || splits < 1, "gemm_tcgen05_decode: %d slices of %d blocks of k", splits, p.k_blocks);
    TI_REQUIRE(p.splits == 1 || epilogue == EPI_PARTIAL, "gemm_tcgen05_decode: a split product leaves partial sums");
    p.halves = n > BMT ? 2 : 1;
    p.stages = stages_for(nt, p.halves);
    TI_REQUIRE(p.stages >= 2, "gemm_tcgen05_decode: tile width %d leaves no room for a pipeline", nt);
    p.stage_bytes = p.halves * A_BYTES + nt * BK * 2;
    p.tmem_cols = 32;
    while (p.tmem_cols < p.halves * nt) p.tmem_cols *= 2;
    p.rotate = 1;                                                // the blocks do not all ask L2 for the same token lines at once
    p.acc_stride = p.halves == 2 ? p.tmem_cols / 2 : 0;          // a power of two of at least nt columns
    p.ldy = ldy; p.epilogue = epilogue; p.act = XieluParams{alpha_p, alpha_n, beta, eps}; p.status = status;
    CUtensorMap mw, mx;
    if (int rc = tensor_map_2d(&mw, W, out, in, in, nt)) return rc;
    if (int rc = tensor_map_2d(&mx, x, n, in, ldx, BMT)) return rc;
    const size_t smem = (size_t)p.stages * p.stage_bytes + 1024 + 256;
    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT);
        if (e != cudaSuccess) return ti_fail("gemm_tcgen05_decode: %s", cudaGetErrorString(e));
        configured = SMEM_LIMIT;
    }
    const int tiles = p.m_tiles * p.splits;
    ti_launch(gemm_tcgen05_decode_kernel, dim3(tiles < sm_count ? tiles : sm_count), dim3(THREADS), smem, stream, mw, mx, y, p);
    return ti_check_launch("gemm_tcgen05_decode");
}
