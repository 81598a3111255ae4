// Causal flash attention for prompts on the Blackwell tensor cores (sm_100a): S = Q Kᵀ and O += P V are
// tcgen05.mma with accumulators in tensor memory, K and V pages come straight from the paged cache
// by TMA, and the softmax runs one thread per query row on the accumulator read back with tcgen05.ld.
//
// A block serves one KV head of one sequence and TWO query tiles of 128 rows each (a row is a
// (token, query head of the group) pair, so the heads of a group share the K and V they read). Warps 0-3
// are the softmax of tile 0, warps 4-7 of tile 1; one thread of warp 8 loads (TMA), one thread of warp 9
// issues the MMAs of both tiles in turn (a tile's two products back to back: issued from two threads
// they would share the tensor core and both finish late). While the softmax of one tile runs, the tensor core works on the other tile. Per step of 128 keys:
//   S_x = Q_x Kᵀ              (SS MMA, both operands K-major in 128-byte-swizzled shared memory)
//   softmax: row maximum, p = 2^(s·c − m) in 32-bit, row sum; P rounded to bfloat16 and written over
//            S in tensor memory
//   O_x += P_x V              (A = P from tensor memory, B = V MN-major: V lies [key][d] as in the cache)
// The running maximum m is only raised (and O rescaled, in tensor memory) when a row's maximum grows by
// more than 2^8: p then stays below 2^8, which bfloat16 and the 32-bit sums carry without loss.
//
// Every wait on an mbarrier is bounded: after the limit the kernel records a code in `status`, stops
// issuing work, frees its tensor memory and returns.
//
// AntoineBut/TileInfer.jl's counterpart is its flash-attention tile kernel (src/ops/tile/attention.jl):
// scores, softmax statistics and sums in 32-bit, P rounded to the storage type for the second product.
#include "tcgen05.cuh"
#include "tensor_map.h"

namespace {

using namespace tc;

constexpr int ROWS = 128;            // rows of a query tile (tensor-memory lanes)
constexpr int KEYS = 128;            // keys per step
constexpr int PAGE = 64;             // keys per cache page
constexpr int RING = 4;              // K and V tiles in flight (K_j, V_j, K_j+1, V_j+1)
constexpr int THREADS = 320;
constexpr float RESCALE_STEP = 8.f;  // in log2 units

struct Params {
    bf16* out;
    const int* table; long long table_stride;
    const int* slots; const int* cu_seqlens; const int* kv_lens;
    int n_seqs, heads, kv_heads, group, window;
    float scale_log2;
    int* status;
};

template <int D> struct Cfg {
    static constexpr int HALVES = D / 64;                       // 64-element (128-byte) column blocks of a row
    static constexpr int Q_TILE_BYTES = ROWS * D * 2;
    static constexpr int KV_TILE_BYTES = KEYS * D * 2;
    static constexpr int HALF_BYTES = 128 * 128;                // 128 rows of 128 bytes
    static constexpr size_t SMEM = 2 * Q_TILE_BYTES + RING * KV_TILE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
    static constexpr int TMEM_COLS = 512;                       // S0 S1 (128 each), O0 O1 (D each)
    static constexpr int O_COL = 256;
};

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Two 32-bit floats in one 64-bit register, for the packed FMA-pipe instructions of sm_100 (one issue
// slot for two lanes of work).
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float a, float b) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
template <int D>
__global__ void __launch_bounds__(THREADS, 1) attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                          const __grid_constant__ CUtensorMap map_k,
                                                                          const __grid_constant__ CUtensorMap map_v,
                                                                          const bf16* q, Params p) {
    typedef Cfg<D> C;
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
    unsigned char* q_tiles = smem;
    unsigned char* kv_tiles = smem + 2 * C::Q_TILE_BYTES;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(kv_tiles + RING * C::KV_TILE_BYTES);
    const unsigned q_full = smem_addr(bars), kv_full0 = q_full + 8, kv_empty0 = kv_full0 + 8 * RING;
    const unsigned s_full0 = kv_empty0 + 8 * RING, p_ready0 = s_full0 + 16, o_done0 = p_ready0 + 16;
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 1 + 2 * RING + 6);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Blocks are numbered so that the hardware hands them out longest first: the block index within
    // the sequences is the slow digit (reversed below), the KV head the fast one.
    const int kvh = blockIdx.x % p.kv_heads;
    const int tokens_per_tile = ROWS / p.group;
    const int tokens_per_block = 2 * tokens_per_tile;

    pdl_wait();
    pdl_launch_dependents();

    // Which sequence and which block of its new tokens; later blocks (longer prefixes) run first.
    int b = 0, blk = (int)(gridDim.x / p.kv_heads) - 1 - (int)(blockIdx.x / p.kv_heads);
    for (; b < p.n_seqs; ++b) {
        const int n_b = (__ldcg(p.cu_seqlens + b + 1) - __ldcg(p.cu_seqlens + b) + tokens_per_block - 1) / tokens_per_block;
        if (blk < n_b) break;
        blk -= n_b;
    }
    if (b >= p.n_seqs) return;
    const int tok_begin = __ldcg(p.cu_seqlens + b), q_len = __ldcg(p.cu_seqlens + b + 1) - tok_begin;
    const int kv_len = __ldcg(p.kv_lens + b), slot = __ldcg(p.slots + b);
    const int start = kv_len - q_len;                           // position of the sequence's first new token
    const int t0 = blk * tokens_per_block;                      // first token of the block among the new ones
    const int t_end = min(q_len, t0 + tokens_per_block);
    // Keys [key_lo, key_hi) can matter to some row of the block.
    const int key_hi = start + t_end;
    const int key_lo = p.window > 0 ? max(0, start + t0 - p.window + 1) : 0;
    const int j_lo = key_lo / KEYS, j_hi = (key_hi + KEYS - 1) / KEYS;
    const int n_pages = (kv_len + PAGE - 1) / PAGE;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < RING; ++s) { mbar_init(kv_full0 + 8 * s, 1); mbar_init(kv_empty0 + 8 * s, 1); }
        for (int x = 0; x < 2; ++x) { mbar_init(s_full0 + 8 * x, 1); mbar_init(p_ready0 + 8 * x, 4); mbar_init(o_done0 + 8 * x, 1); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 9) tmem_alloc(smem_addr(tmem_slot), C::TMEM_COLS);
    // A group that does not divide 128 leaves the last rows of a query tile without a (token, head): the TMA box does not
    // write them, so they are zeroed here once (whole 128-byte rows: the swizzle moves bytes within a row only), and
    // nothing is written out for them below.
    const int rows_used = tokens_per_tile * p.group;
    if (rows_used < ROWS) {
        const int spare = ROWS - rows_used, words = spare * 32;         // 32 words of 4 bytes a row
        for (int i = threadIdx.x; i < 2 * C::HALVES * words; i += THREADS) {
            const int blk = i / words, w = i % words;                    // blk: (tile, 64-column block)
            reinterpret_cast<unsigned*>(q_tiles + (size_t)blk * C::HALF_BYTES + (size_t)rows_used * 128)[w] = 0u;
        }
        fence_async_smem();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *tmem_slot;

    if (warp == 8) {
        // ---------------------------------------------------------------- loads (one thread)
        if (lane == 0) {
            mbar_expect_tx(q_full, (unsigned)(2 * rows_used * D * 2));
            for (int x = 0; x < 2; ++x)
                for (int h = 0; h < C::HALVES; ++h)
                    tma_load_3d(smem_addr(q_tiles + x * C::Q_TILE_BYTES + h * C::HALF_BYTES), &map_q, h * 64, kvh * p.group,
                                tok_begin + t0 + x * tokens_per_tile, q_full);
            // A page past the sequence's last one is replaced by the last one: its keys are masked, but
            // what stands in shared memory must be finite.
            const int* table = p.table + (long long)slot * p.table_stride;
            int page[KEYS / PAGE], next_page[KEYS / PAGE];
            for (int pg = 0; pg < KEYS / PAGE; ++pg) page[pg] = __ldcg(table + min(j_lo * (KEYS / PAGE) + pg, n_pages - 1));
            bool ok = true;
            int fill = 0;                                       // K_j is fill 2(j - j_lo), V_j the next one
            for (int j = j_lo; ok && j < j_hi; ++j) {
                // The next step's page numbers are on their way while this step's tiles are waited for.
                for (int pg = 0; pg < KEYS / PAGE; ++pg)
                    next_page[pg] = j + 1 < j_hi ? __ldcg(table + min((j + 1) * (KEYS / PAGE) + pg, n_pages - 1)) : 0;
                for (int kv = 0; kv < 2; ++kv, ++fill) {
                    const int buf = fill % RING;
                    const unsigned phase = (unsigned)(fill / RING) & 1u;
                    ok = mbar_wait(kv_empty0 + 8 * buf, phase ^ 1, p.status, 1);
                    if (!ok) break;
                    const unsigned bar = kv_full0 + 8 * buf;
                    mbar_expect_tx(bar, C::KV_TILE_BYTES);
                    const unsigned dst = smem_addr(kv_tiles + (size_t)buf * C::KV_TILE_BYTES);
                    for (int pg = 0; pg < KEYS / PAGE; ++pg) {
                        const int row = (page[pg] * p.kv_heads + kvh) * PAGE;
                        for (int h = 0; h < C::HALVES; ++h)
                            tma_load_2d(dst + h * C::HALF_BYTES + pg * (PAGE * 128), kv ? &map_v : &map_k, h * 64, row, bar);
                    }
                }
                for (int pg = 0; pg < KEYS / PAGE; ++pg) page[pg] = next_page[pg];
            }
        }
    } else if (warp == 9) {
        // ---------------------------------------------------------------- MMA issue (one thread)
        if (lane == 0) {
            constexpr unsigned IDESC_QK = instr_desc_bf16(ROWS, KEYS, false);
            constexpr unsigned IDESC_PV = instr_desc_bf16(ROWS, D, true);
            // S_x = Q_x K_jᵀ into tensor-memory columns [128 x, 128 x + 128).
            auto issue_qk = [&](int x, int buf) {
                const unsigned qa = smem_addr(q_tiles + x * C::Q_TILE_BYTES);
                const unsigned ka = smem_addr(kv_tiles + (size_t)buf * C::KV_TILE_BYTES);
#pragma unroll
                for (int s = 0; s < D / 16; ++s) {
                    const unsigned off = (s / 4) * C::HALF_BYTES + (s % 4) * 32;
                    umma_bf16(tmem_base + x * KEYS, smem_desc_sw128(qa + off), smem_desc_sw128(ka + off), IDESC_QK, s > 0 ? 1u : 0u);
                }
                umma_commit(s_full0 + 8 * x);
            };
            bool ok = mbar_wait(q_full, 0, p.status, 2);
            if (ok && j_lo < j_hi) {
                ok = mbar_wait(kv_full0, 0, p.status, 3);
                tc_fence_after();
                if (ok) {
                    issue_qk(0, 0);
                    issue_qk(1, 0);
                    umma_commit(kv_empty0);
                }
            }
            int fill = 0;
            for (int j = j_lo; ok && j < j_hi; ++j, fill += 2) {
                const int vbuf = (fill + 1) % RING, knext = (fill + 2) % RING;
                const unsigned vphase = (unsigned)((fill + 1) / RING) & 1u, kphase = (unsigned)((fill + 2) / RING) & 1u;
                const unsigned jphase = (unsigned)(j - j_lo) & 1u;
                ok = mbar_wait(kv_full0 + 8 * vbuf, vphase, p.status, 4);
                if (ok && j + 1 < j_hi) ok = mbar_wait(kv_full0 + 8 * knext, kphase, p.status, 6);
                if (!ok) break;
                const unsigned va = smem_addr(kv_tiles + (size_t)vbuf * C::KV_TILE_BYTES);
                for (int x = 0; x < 2; ++x) {
                    ok = mbar_wait(p_ready0 + 8 * x, jphase, p.status, 5);
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int s = 0; s < KEYS / 16; ++s)         // 16 keys = 16 rows of 128 bytes further on
                        umma_bf16_ts(tmem_base + C::O_COL + x * D, tmem_base + x * KEYS + s * 8,
                                     smem_desc_mn_sw128(va + s * 2048, C::HALF_BYTES, 1024), IDESC_PV, (j > j_lo || s > 0) ? 1u : 0u);
                    umma_commit(o_done0 + 8 * x);
                    if (j + 1 < j_hi) issue_qk(x, knext);
                }
                if (!ok) break;
                umma_commit(kv_empty0 + 8 * vbuf);
                if (j + 1 < j_hi) umma_commit(kv_empty0 + 8 * knext);
            }
        }
    } else {
        // ---------------------------------------------------------------- softmax, one thread per row
        const int x = warp >> 2;                                // query tile
        const int row = (warp & 3) * 32 + lane;                 // tensor-memory lane
        const int tok = t0 + x * tokens_per_tile + row / p.group;
        const int head = kvh * p.group + row % p.group;
        const int pos = start + tok;
        const int warp_pos_lo = start + t0 + x * tokens_per_tile + ((warp & 3) * 32) / p.group;   // smallest position in the warp
        const int warp_pos_hi = start + t0 + x * tokens_per_tile + ((warp & 3) * 32 + 31) / p.group;
        const unsigned lane_base = tmem_base + ((unsigned)((warp & 3) * 32) << 16);
        const unsigned s_addr = lane_base + x * KEYS, o_addr = lane_base + C::O_COL + x * D;
        float m_used = -1e30f, l = 0.f;
        bool ok = true;
        for (int j = j_lo; ok && j < j_hi; ++j) {
            const unsigned jphase = (unsigned)(j - j_lo) & 1u;
            ok = __all_sync(0xffffffffu, mbar_wait(s_full0 + 8 * x, jphase, p.status, 7));
            if (!ok) break;
            tc_fence_after();
            const int key0 = j * KEYS;
            // Warp-uniform: does any row of this warp have a masked key in this step?
            const bool masked = key0 + KEYS - 1 > warp_pos_lo || (p.window > 0 && key0 <= warp_pos_hi - p.window);
            const int k_hi = pos, k_lo = p.window > 0 ? pos - p.window + 1 : 0;        // the row sees keys [k_lo, k_hi]
            // The whole row of scores in registers: four loads in flight, one wait.
            unsigned r[4][32];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld32(s_addr + c * 32, r[c]);
            tmem_ld_wait();
            if (masked) {
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int key = key0 + c * 32 + i;
                        if (!(key <= k_hi && key >= k_lo)) r[c][i] = 0xff800000u;       // -inf: its weight is exactly zero
                    }
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // independent chains
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(r[c][i]));
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            const float mt = fmaxf(mx * p.scale_log2, -1e30f);
            if (j == j_lo) {
                m_used = mt;
            } else if (__any_sync(0xffffffffu, mt > m_used + RESCALE_STEP)) {
                // O must be complete (the previous step's second product) before it is rescaled.
                ok = __all_sync(0xffffffffu, mbar_wait(o_done0 + 8 * x, jphase ^ 1, p.status, 8));
                if (!ok) break;
                tc_fence_after();
                const float m_new = fmaxf(m_used, mt);
                const float alpha = ex2(m_used - m_new);
                l *= alpha;
                m_used = m_new;
#pragma unroll 1
                for (int c = 0; c < D / 32; ++c) {
                    unsigned o[32];
                    tmem_ld32(o_addr + c * 32, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tmem_st32(o_addr + c * 32, o);
                }
                tmem_st_wait();
            }
            f32x2 l2[2] = {0ull, 0ull};                          // two chains of packed sums
            const f32x2 scale2 = pack2(p.scale_log2, p.scale_log2), neg_m2 = pack2(-m_used, -m_used);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                unsigned packed[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    const f32x2 x2 = fma2(pack2(__uint_as_float(r[c][i]), __uint_as_float(r[c][i + 1])), scale2, neg_m2);
                    float p0, p1;
                    unpack2(x2, p0, p1);
                    p0 = ex2(p0);
                    p1 = ex2(p1);
                    l2[(i >> 1) & 1] = add2(l2[(i >> 1) & 1], pack2(p0, p1));
                    const __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
                    packed[i / 2] = *reinterpret_cast<const unsigned*>(&pk);
                }
                tmem_st16(s_addr + c * 16, packed);             // P over S, which is in registers by now
            }
            {
                float a0, a1, b0, b1;
                unpack2(l2[0], a0, a1);
                unpack2(l2[1], b0, b1);
                l += (a0 + a1) + (b0 + b1);
            }
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_ready0 + 8 * x);
        }
        if (ok && j_lo < j_hi) {
            ok = __all_sync(0xffffffffu, mbar_wait(o_done0 + 8 * x, (unsigned)(j_hi - 1 - j_lo) & 1u, p.status, 9));
            tc_fence_after();
        }
        if (ok) {
            const float inv = l > 0.f ? 1.f / l : 0.f;
            bf16* dst = p.out + ((size_t)(tok_begin + tok) * p.heads + head) * D;
#pragma unroll 1
            for (int c = 0; c < D / 32; ++c) {
                unsigned r[32];
                tmem_ld32(o_addr + c * 32, r);
                tmem_ld_wait();
                if (tok < q_len && row < rows_used) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 w;
                        unsigned* wp = reinterpret_cast<unsigned*>(&w);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(r[i + 2 * e]) * inv, __uint_as_float(r[i + 2 * e + 1]) * inv);
                            wp[e] = *reinterpret_cast<const unsigned*>(&h2);
                        }
                        *reinterpret_cast<uint4*>(dst + c * 32 + i) = w;
                    }
                }
            }
        }
    }
    if (*reinterpret_cast<volatile int*>(p.status) != 0) drain_after_timeout();   // a wait ran out somewhere: let what is in flight land
    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

template <int D>
int launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const bf16* q, const Params& p, int blocks,
           cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<D>::SMEM);
        if (e != cudaSuccess) return ti_fail("attention_prefill_tc: %s", cudaGetErrorString(e));
        configured = true;
    }
    ti_launch(attention_prefill_tc_kernel<D>, dim3(blocks * p.kv_heads), dim3(THREADS), Cfg<D>::SMEM, stream, mq, mk, mv, q, p);
    return ti_check_launch("attention_prefill_tc");
}

}  // namespace

// out, q: [tokens, nq, D] bfloat16; k_cache, v_cache: [pages, nkv, 64, D] bfloat16. `total_blocks` = sum over
// the sequences of ceil(new tokens / (2 * (128 / (nq / nkv)))), the division inside rounding down. `status` is a device word that must be zero; a
// non-zero value afterwards means a wait ran out. Returns 2 when the sizes are outside what this kernel
// takes (head size 64 or 128, 1 to 128 query heads per KV head, pages of 64): the caller then runs the
// kernel for all sizes.
extern "C" int ti_attention_prefill_tc(void* out, const void* q, const void* k_cache, const void* v_cache, int n_pages,
                                       const int* block_table, int table_stride, const int* seq_slots,
                                       const int* cu_seqlens, const int* kv_lens, int n_seqs, int n_tokens, int total_blocks,
                                       float scale, int nq, int nkv, int D, int page_size, int window, int* status,
                                       cudaStream_t stream) {
    if (n_seqs == 0 || total_blocks == 0) return 0;
    const int group = nkv > 0 ? nq / nkv : 0;
    if (page_size != PAGE || nkv <= 0 || nq % nkv != 0 || group < 1 || group > ROWS || (D != 64 && D != 128) || nkv > 65535 ||
        ((uintptr_t)q & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15) || ((uintptr_t)out & 15)) {
        ti_fail("attention_prefill_tc takes head size 64 or 128, pages of 64 and 1 to 128 query heads per KV head; "
                "got head size %d, page %d, %d/%d heads", D, page_size, nq, nkv);
        return 2;
    }
    TI_REQUIRE(status != nullptr, "attention_prefill_tc: status word missing");
    Params p;
    p.out = (bf16*)out; p.table = block_table; p.table_stride = table_stride; p.slots = seq_slots; p.cu_seqlens = cu_seqlens;
    p.kv_lens = kv_lens; p.n_seqs = n_seqs; p.heads = nq; p.kv_heads = nkv; p.group = group; p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
    CUtensorMap mq, mk, mv;
    {
        const unsigned long long dims[3] = {(unsigned long long)D, (unsigned long long)nq, (unsigned long long)n_tokens};
        const unsigned long long strides[2] = {(unsigned long long)D * 2, (unsigned long long)nq * D * 2};
        const unsigned box[3] = {64, (unsigned)group, (unsigned)(ROWS / group)};
        if (int rc = ti_tensor_map_bf16(&mq, q, 3, dims, strides, box, true)) return rc;
    }
    {
        const unsigned long long dims[2] = {(unsigned long long)D, (unsigned long long)n_pages * nkv * PAGE};
        const unsigned long long strides[1] = {(unsigned long long)D * 2};
        const unsigned box[2] = {64, PAGE};
        if (int rc = ti_tensor_map_bf16(&mk, k_cache, 2, dims, strides, box, true)) return rc;
        if (int rc = ti_tensor_map_bf16(&mv, v_cache, 2, dims, strides, box, true)) return rc;
    }
    return D == 64 ? launch<64>(mq, mk, mv, (const bf16*)q, p, total_blocks, stream)
                   : launch<128>(mq, mk, mv, (const bf16*)q, p, total_blocks, stream);
}
