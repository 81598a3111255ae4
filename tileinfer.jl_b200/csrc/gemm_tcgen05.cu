// Tensor-core matrix product for sm_100a: y[n, out] = x[n, in] · W[out, in]ᵀ in bfloat16 with
// 32-bit accumulation, written directly against the Blackwell instructions: TMA
// (cp.async.bulk.tensor) stages both operands in 128-byte-swizzled shared memory,
// tcgen05.mma (issued by one thread) accumulates in tensor memory, tcgen05.ld brings the
// accumulator back for the epilogue.
//
// The WEIGHTS are the 128-row operand and the tokens the N operand (16 to 256 wide), so the
// same kernel serves prefill (N = 256 tokens per tile) and decode batches (N = the batch),
// where it is a weight-streaming kernel whose TMA pipeline keeps ~190 KB in flight per SM.
// Both operands are K-major exactly as they lie in memory ([out, in] weights, [n, in]
// activations): no transposes anywhere.
//
// One persistent block per SM walks output tiles (token tile fastest, so the blocks that
// run together share weight tiles in L2). Warp 0 produces (TMA), warp 1 issues the MMAs,
// warps 2-9 run the epilogue on one of two accumulator buffers in tensor memory while the
// MMAs of the next tile fill the other. A product with few output tiles can be split over
// k; the 32-bit partial sums [split, n, out] are added by the residual-add + RMSNorm kernel.
// Epilogues: round to bfloat16; xIELU on the rounded sums; 32-bit logits; raw partials.
// bfloat16 results of wide token tiles are transposed through shared memory and leave by TMA stores
// (64-byte rows instead of 2 bytes per thread; measured 274 -> 250 us on 21504 x 4096 x 2048 tokens).
//
// Every wait on an mbarrier is bounded: after the limit the kernel records a code in
// `status`, stops issuing work, frees its tensor memory and returns.
//
// AntoineBut/TileInfer.jl's counterpart is gemm_kernel (src/ops/tile/linear.jl:80-100): 32-bit
// accumulation, one rounding to the storage type, grouped tile order for L2 reuse.
#include "tcgen05.cuh"
#include "tensor_map.h"


namespace {

using namespace tc;

constexpr int BM = 128;            // weight rows per tile (tensor-memory lanes)
constexpr int BK = 64;             // k per stage: 64 bf16 = one 128-byte swizzle row
// Epilogue warps: 8 (two per tensor-memory lane quarter, each takes every other column chunk) for wide
// token tiles; 4 for token tiles of up to 64, whose blocks are small enough for TWO to share an SM, so
// that a product with a few more tiles than SMs does not pay for a second wave.
constexpr int SMEM_LIMIT = 227 * 1024;
constexpr int OUT_TILE_BYTES = 32 * 32 * 2;   // a staging tile of 32 tokens x 32 features

enum { EPI_NONE = 0, EPI_XIELU = 1, EPI_F32 = 2, EPI_PARTIAL = 3 };

struct Params {
    int M, N, K;                   // out features, tokens, in features
    int m_tiles, n_tiles, splits, k_blocks;
    long long ldy;
    int epilogue;
    XieluParams act;
    int* status;
    int tma_out;                   // bfloat16 results leave through shared memory and TMA stores
    int rotate;                    // every weight tile starts at another place of its k range
};

// MT: 128-row weight sub-tiles per block. With MT = 2 a block owns 256 weight rows: the token
// operand staged for a k block feeds two MMAs, so a k block moves 64 KB for 1024 tensor-core cycles
// instead of 48 KB for 512, which is what the L2 -> shared-memory path can sustain. Both accumulators
// then fill tensor memory (2 x 256 columns), so the epilogue of a tile is not overlapped with the next
// tile's MMAs; it is about a tenth of a tile's time.
template <int BN, int MT> struct Cfg {
    static constexpr int BLOCKS_PER_SM = BN <= 64 ? 2 : 1;
    static constexpr int EPI_WARPS = BN <= 64 ? 4 : 8;
    static constexpr int THREADS = 64 + 32 * EPI_WARPS;
    static constexpr int A_BYTES = MT * BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    // Wide token tiles write bfloat16 results through shared memory: each epilogue warp owns two
    // staging tiles of 32 tokens x 32 features that leave by TMA stores.
    static constexpr int OUT_BYTES = BN >= 128 ? EPI_WARPS * 2 * OUT_TILE_BYTES : 0;
    static constexpr int STAGES_FIT = (SMEM_LIMIT / BLOCKS_PER_SM - 2048 - OUT_BYTES) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_FIT > 8 ? 8 : STAGES_FIT;
    static constexpr int ACC_BUFS = MT == 2 ? 1 : 2;
    static constexpr int TMEM_COLS = ACC_BUFS * MT * BN < 32 ? 32 : ACC_BUFS * MT * BN;
    static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + OUT_BYTES + 1024 /*alignment slack*/ + 512 /*barriers*/;
};

// kind::f16 instruction descriptor: D 32-bit, A and B bfloat16, both K-major, M = 128, N = BN.
template <int BN> __device__ __forceinline__ constexpr unsigned instr_desc() {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(BM >> 4) << 24);
}

struct TileIter {
    int id, step, total;
    int m, n, kb_lo, kb_hi, split, rot;
    __device__ bool next(const Params& p) {
        if (id >= total) return false;
        int t = id;
        n = t % p.n_tiles; t /= p.n_tiles;
        split = t % p.splits; m = t / p.splits;
        kb_lo = (int)((long long)p.k_blocks * split / p.splits);
        kb_hi = (int)((long long)p.k_blocks * (split + 1) / p.splits);
        rot = p.rotate ? (m * 7) % (kb_hi - kb_lo) : 0;
        id += step;
        return true;
    }
    __device__ int kb_at(int i) const { const int n_kb = kb_hi - kb_lo; int k = i + rot; if (k >= n_kb) k -= n_kb; return kb_lo + k; }
};

// The epilogue of 32 accumulator rows (one warp's tensor-memory lanes, features m_first .. m_first + 31)
// over the token columns of a tile: every (EPI_WARPS / 4)-th chunk of 32 columns, starting at col_group.
template <int BN, int EPI_WARPS, int OUT_BYTES>
__device__ __forceinline__ void epilogue_rows(unsigned t_row, int m_first, int lane, int n0, int n_valid, int col_group, int warp_slot,
                                              int split, int& out_buf, unsigned char* out_tiles, const CUtensorMap* map_y, void* y,
                                              const Params& p, const XieluPacked& act) {
    constexpr int CH = BN >= 32 ? 32 : 16;
    const int m = m_first + lane;
#pragma unroll 1
    for (int c = col_group * CH; c < BN; c += (EPI_WARPS / 4) * CH) {
        if (c >= n_valid) break;                   // uniform across the warp
        unsigned r[32];
        if (CH == 32) tmem_ld32(t_row + c, r); else tmem_ld16(t_row + c, r);
        tmem_ld_wait();
        // All values of the chunk first, without branches (one warp per scheduler runs this: only
        // independent elements in flight hide the latency of the arithmetic), then the stores.
        if (p.epilogue >= EPI_F32) {
            if (m < p.M) {
                float* yf = (float*)y + ((size_t)(p.epilogue == EPI_PARTIAL ? split : 0) * p.N + n0 + c) * p.ldy + m;
#pragma unroll
                for (int j = 0; j < CH; ++j) {
                    const float s = __uint_as_float(r[j]);
                    if (c + j < n_valid) yf[(size_t)j * p.ldy] = p.epilogue == EPI_PARTIAL ? s : rnd<bf16>(s);
                }
            }
            continue;
        }
        unsigned o[32];                            // bfloat16 bits in the low halves
#pragma unroll
        for (int j = 0; j < CH; j += 2) {
            const float s0 = __uint_as_float(r[j]), s1 = __uint_as_float(r[j + 1]);
            if (p.epilogue == EPI_XIELU) {
                xielu_bf16_pair(s0, s1, act, o[j], o[j + 1]);
            } else {
                const __nv_bfloat162 q = __floats2bfloat162_rn(s0, s1);
                const unsigned bits = *reinterpret_cast<const unsigned*>(&q);
                o[j] = bits & 0xffffu; o[j + 1] = bits >> 16;
            }
        }
        if (OUT_BYTES > 0 && p.tma_out) {
            // The warp's 32 features x 32 tokens go to one of its two staging tiles ([token][feature],
            // so a warp writes 64 contiguous bytes at a time) and leave as one TMA store, which
            // writes whole 64-byte rows instead of 2 bytes per thread.
            unsigned char* tile = out_tiles + (size_t)((warp_slot * 2 + out_buf) * OUT_TILE_BYTES);
            if (lane == 0) tma_store_wait_read<1>();          // the store that last read this tile has done so
            __syncwarp();
#pragma unroll
            for (int j = 0; j < CH; ++j)
                reinterpret_cast<unsigned short*>(tile)[j * 32 + lane] = (unsigned short)o[j];
            fence_async_smem();
            __syncwarp();
            if (lane == 0 && m_first < p.M) tma_store_2d(map_y, smem_addr(tile), m_first, n0 + c);
            out_buf ^= 1;
        } else if (m < p.M) {
            unsigned short* yb = (unsigned short*)y + (size_t)(n0 + c) * p.ldy + m;
#pragma unroll
            for (int j = 0; j < CH; ++j)
                if (c + j < n_valid) yb[(size_t)j * p.ldy] = (unsigned short)o[j];
        }
    }
}

template <int BN, int MT>
__global__ void __launch_bounds__(Cfg<BN, MT>::THREADS, Cfg<BN, MT>::BLOCKS_PER_SM) gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                 const __grid_constant__ CUtensorMap map_x,
                                                                 const __grid_constant__ CUtensorMap map_y,
                                                                 void* __restrict__ y, Params p) {
    typedef Cfg<BN, MT> C;
    extern __shared__ unsigned char smem_dyn[];
    // Swizzled tiles need 1024-byte alignment.
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
    unsigned char* tiles = smem;
    unsigned char* out_tiles = smem + (size_t)C::STAGES * C::STAGE_BYTES;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(out_tiles + C::OUT_BYTES);
    // bars: full[STAGES], empty[STAGES], acc_full[2], acc_empty[2]; then the tensor-memory base address.
    const unsigned full0 = smem_addr(bars), empty0 = full0 + 8 * C::STAGES;
    const unsigned accf0 = empty0 + 8 * C::STAGES, acce0 = accf0 + 16;
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 2 * C::STAGES + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(accf0 + 8 * a, 1); mbar_init(acce0 + 8 * a, C::EPI_WARPS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_addr(tmem_slot), C::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    TileIter it;
    it.id = blockIdx.x; it.step = gridDim.x; it.total = p.m_tiles * p.n_tiles * p.splits;

    // Barriers and tensor memory are set up while the previous kernel drains, and the weights do not
    // depend on it: the loads of the first tile's first weight blocks (as many as the pipeline has
    // stages) are on their way before the wait. The previous kernel's results (the activations, and the
    // output buffer it may still read) are touched only after it.
    int ahead = 0;
    if (warp == 0) {
        TileIter first = it;
        if (first.next(p)) {
            ahead = min(C::STAGES, first.kb_hi - first.kb_lo);
            if (lane == 0)
                for (int s = 0; s < ahead; ++s) {
                    const unsigned bar = full0 + 8 * s;
                    mbar_expect_tx(bar, C::STAGE_BYTES);
                    const unsigned a_dst = smem_addr(tiles + (size_t)s * C::STAGE_BYTES);
#pragma unroll
                    for (int h = 0; h < MT; ++h)
                        tma_load_2d(a_dst + h * (BM * BK * 2), &map_w, first.kb_at(s) * BK, (first.m * MT + h) * BM, bar);
                }
            __syncwarp();
        }
    }
    pdl_wait();
    pdl_launch_dependents();
    const unsigned tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------------------------------------------------------- producer (TMA)
        // ONE thread walks the loop: a wait that the whole warp executes costs 32 barrier tests and a vote
        // per k block, which at 64 of k per stage is more than the copy it guards.
        int stage = 0;
        unsigned phase = 0;
        bool ok = true;
        int issued = 0;                                     // k blocks of this block so far
        while (lane == 0 && ok && it.next(p)) {
            for (int i = 0; i < it.kb_hi - it.kb_lo; ++i, ++issued) {
                const int kb = it.kb_at(i);
                ok = mbar_wait(empty0 + 8 * stage, phase ^ 1, p.status, 1);
                if (!ok) break;
                const unsigned bar = full0 + 8 * stage;
                const unsigned a_dst = smem_addr(tiles + (size_t)stage * C::STAGE_BYTES);
                if (issued >= ahead) {                      // else the weights of this stage are already on their way
                    mbar_expect_tx(bar, C::STAGE_BYTES);
#pragma unroll
                    for (int h = 0; h < MT; ++h)
                        tma_load_2d(a_dst + h * (BM * BK * 2), &map_w, kb * BK, (it.m * MT + h) * BM, bar);
                }
                tma_load_2d(a_dst + C::A_BYTES, &map_x, kb * BK, it.n * BN, bar);
                if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer (one thread)
        int stage = 0;
        unsigned phase = 0;
        int local = 0;
        bool ok = true;
        while (lane == 0 && ok && it.next(p)) {
            const int acc = C::ACC_BUFS == 2 ? (local & 1) : 0;
            const unsigned acc_phase = C::ACC_BUFS == 2 ? ((local >> 1) & 1) : (local & 1);
            ok = mbar_wait(acce0 + 8 * acc, acc_phase ^ 1, p.status, 2);
            if (!ok) break;
            tc_fence_after();
            const unsigned d_tmem = tmem_base + (unsigned)(acc * MT * BN);
            for (int i = 0; i < it.kb_hi - it.kb_lo; ++i) {
                ok = mbar_wait(full0 + 8 * stage, phase, p.status, 3);
                if (!ok) break;
                tc_fence_after();
                const unsigned a_addr = smem_addr(tiles + (size_t)stage * C::STAGE_BYTES);
                const unsigned long long db = smem_desc_sw128(a_addr + C::A_BYTES);
#pragma unroll
                for (int k = 0; k < BK / 16; ++k)          // 16 k = 32 bytes further along the swizzled row
#pragma unroll
                    for (int h = 0; h < MT; ++h)           // the sub-tiles share the token operand
                        umma_bf16(d_tmem + (unsigned)(h * BN), smem_desc_sw128(a_addr + h * (BM * BK * 2)) + (unsigned long long)(2 * k),
                                  db + (unsigned long long)(2 * k), instr_desc<BN>(), (i > 0 || k > 0) ? 1u : 0u);
                umma_commit(empty0 + 8 * stage);           // the stage is free once these MMAs have read it
                if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
            }
            if (!ok) break;
            umma_commit(accf0 + 8 * acc);                  // the accumulator is complete
            ++local;
        }
    } else {
        // ---------------------------------------------------------------- epilogue (4 or 8 warps)
        const int quarter = warp & 3;                      // the tensor-memory lanes this warp may read
        const int col_group = (warp - 2) >> 2;             // with 8 warps the chunks of columns alternate between two warps
        int local = 0, out_buf = 0;
        const XieluPacked act = xielu_pack(p.act);
        bool ok = true;
        while (ok && it.next(p)) {
            const int acc = C::ACC_BUFS == 2 ? (local & 1) : 0;
            const unsigned acc_phase = C::ACC_BUFS == 2 ? ((local >> 1) & 1) : (local & 1);
            ok = __all_sync(0xffffffffu, mbar_wait(accf0 + 8 * acc, acc_phase, p.status, 4));
            if (!ok) break;
            tc_fence_after();
            const int n0 = it.n * BN;
            const int n_valid = min(BN, p.N - n0);
#pragma unroll 1
            for (int h = 0; h < MT; ++h) {
            const int m_first = (it.m * MT + h) * BM + quarter * 32;
            const unsigned t_row = tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)((acc * MT + h) * BN);
            epilogue_rows<BN, C::EPI_WARPS, C::OUT_BYTES>(t_row, m_first, lane, n0, n_valid, col_group, warp - 2, it.split, out_buf,
                                                          out_tiles, &map_y, y, p, act);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acce0 + 8 * acc);
            ++local;
        }
        if (C::OUT_BYTES > 0 && lane == 0) tma_store_wait_all();   // shared memory stays until the stores have read it
    }
    if (*reinterpret_cast<volatile int*>(p.status) != 0) drain_after_timeout();   // a wait ran out somewhere: let what is in flight land
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------ two SMs per tile
// A cluster of two blocks owns a tile of 256 weight rows x 256 tokens with tcgen05.mma.cta_group::2:
// each block stages its own 128 weight rows and HALF of the tokens (the tensor cores read the other
// half from the partner's shared memory), and each block's tensor memory receives its 128 rows of the
// result. 64 of k thus cost each SM 32 KB of shared-memory fill for 512 tensor-core cycles (48 KB with
// one SM per tile), with both accumulator buffers kept, so the epilogue still overlaps the next tile.
// A stage holds 128 of k (64 KB, three stages): one barrier round trip per 1,024 tensor-core cycles.
// Block 0 of the pair issues the MMAs; its `full` barriers count the bytes of both blocks' loads; commits
// arrive on both blocks' barriers; the partner's epilogue warps arrive on block 0's accumulator barrier.
struct PairCfg {
    static constexpr int BN = 256;                     // tokens per tile
    static constexpr int EPI_WARPS = 8;
    static constexpr int THREADS = 64 + 32 * EPI_WARPS;
    static constexpr int KB = 2;                       // 64-wide (one swizzle row) k blocks per stage: 128 of k
    static constexpr int ATOM_BYTES = 128 * BK * 2;    // 128 rows of one swizzle row each
    static constexpr int A_BYTES = KB * ATOM_BYTES;    // this block's 128 weight rows
    static constexpr int B_BYTES = KB * ATOM_BYTES;    // this block's half (128) of the tokens
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int OUT_BYTES = EPI_WARPS * 2 * OUT_TILE_BYTES;
    static constexpr int STAGES = (SMEM_LIMIT - 2048 - OUT_BYTES) / STAGE_BYTES;
    static constexpr int TMEM_COLS = 2 * BN;
    static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + OUT_BYTES + 1024 + 512;
};

__device__ __forceinline__ unsigned cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// The address of this block's shared-memory location `addr` in block `rank` of the cluster.
__device__ __forceinline__ unsigned map_to_block(unsigned addr, unsigned rank) {
    unsigned r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(unsigned cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// TMA load into this block's shared memory whose bytes are counted on a barrier of either block of the pair.
__device__ __forceinline__ void tma_load_2d_pair(unsigned dst, const CUtensorMap* map, int x, int y, unsigned bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(unsigned dst_smem, unsigned cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(unsigned taddr, unsigned cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(unsigned tmem_d, unsigned long long desc_a, unsigned long long desc_b,
                                               unsigned idesc, unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// One arrival on the barrier at this offset in BOTH blocks when every MMA issued so far has completed.
__device__ __forceinline__ void umma_commit_pair(unsigned bar) {
    const unsigned short mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(mask) : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PairCfg::THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                         const __grid_constant__ CUtensorMap map_y, void* __restrict__ y, Params p) {
    typedef PairCfg C;
    constexpr int BN = C::BN;
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
    unsigned char* tiles = smem;
    unsigned char* out_tiles = smem + (size_t)C::STAGES * C::STAGE_BYTES;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(out_tiles + C::OUT_BYTES);
    const unsigned full0 = smem_addr(bars), empty0 = full0 + 8 * C::STAGES;
    const unsigned accf0 = empty0 + 8 * C::STAGES, acce0 = accf0 + 16;
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 2 * C::STAGES + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned rank = cluster_rank();
    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(accf0 + 8 * a, 1); mbar_init(acce0 + 8 * a, 2 * C::EPI_WARPS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc_pair(smem_addr(tmem_slot), C::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                    // the partner's barriers exist before anything arrives on them
    tc_fence_after();
    pdl_wait();
    pdl_launch_dependents();
    const unsigned tmem_base = *tmem_slot;

    TileIter it;
    it.id = blockIdx.x >> 1; it.step = gridDim.x >> 1; it.total = p.m_tiles * p.n_tiles * p.splits;

    if (warp == 0) {
        // ---------------------------------------------------------------- producer (TMA), in both blocks
        int stage = 0;
        unsigned phase = 0;
        bool ok = true;
        while (lane == 0 && ok && it.next(p)) {             // one thread: see the producer of the kernel above
            for (int kb = it.kb_lo; kb < it.kb_hi; ++kb) {
                ok = mbar_wait(empty0 + 8 * stage, phase ^ 1, p.status, 1);
                if (!ok) break;
                if (rank == 0) mbar_expect_tx(full0 + 8 * stage, 2 * C::STAGE_BYTES);
                const unsigned bar = map_to_block(full0 + 8 * stage, 0);
                const unsigned a_dst = smem_addr(tiles + (size_t)stage * C::STAGE_BYTES);
#pragma unroll
                for (int a = 0; a < C::KB; ++a) {
                    tma_load_2d_pair(a_dst + a * C::ATOM_BYTES, &map_w, (kb * C::KB + a) * BK, (it.m * 2 + (int)rank) * BM, bar);
                    tma_load_2d_pair(a_dst + C::A_BYTES + a * C::ATOM_BYTES, &map_x, (kb * C::KB + a) * BK,
                                     it.n * BN + (int)rank * (BN / 2), bar);
                }
                if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer (block 0, lane 0)
        int stage = 0;
        unsigned phase = 0;
        int local = 0;
        bool ok = true;
        constexpr unsigned IDESC = instr_desc_bf16(2 * BM, BN, false);
        while (rank == 0 && lane == 0 && ok && it.next(p)) {
            const int acc = local & 1;
            const unsigned acc_phase = (local >> 1) & 1;
            ok = mbar_wait(acce0 + 8 * acc, acc_phase ^ 1, p.status, 2);
            if (!ok) break;
            tc_fence_after();
            const unsigned d_tmem = tmem_base + (unsigned)(acc * BN);
            for (int kb = it.kb_lo; kb < it.kb_hi; ++kb) {
                ok = mbar_wait(full0 + 8 * stage, phase, p.status, 3);
                if (!ok) break;
                tc_fence_after();
                const unsigned a_addr = smem_addr(tiles + (size_t)stage * C::STAGE_BYTES);
#pragma unroll
                for (int k = 0; k < C::KB * BK / 16; ++k) {            // 16 k = 32 bytes along the swizzled row; 64 k = the next block of rows
                    const unsigned off = (k / 4) * C::ATOM_BYTES + (k % 4) * 32;
                    umma_bf16_pair(d_tmem, smem_desc_sw128(a_addr + off), smem_desc_sw128(a_addr + C::A_BYTES + off), IDESC,
                                   (kb > it.kb_lo || k > 0) ? 1u : 0u);
                }
                umma_commit_pair(empty0 + 8 * stage);      // the stage is free in both blocks once these MMAs have read it
                if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
            }
            if (!ok) break;
            umma_commit_pair(accf0 + 8 * acc);
            ++local;
        }
    } else {
        // ---------------------------------------------------------------- epilogue (8 warps), in both blocks
        const int quarter = warp & 3;
        const int col_group = (warp - 2) >> 2;
        int local = 0, out_buf = 0;
        const XieluPacked act = xielu_pack(p.act);
        bool ok = true;
        while (ok && it.next(p)) {
            const int acc = local & 1;
            const unsigned acc_phase = (local >> 1) & 1;
            ok = __all_sync(0xffffffffu, mbar_wait(accf0 + 8 * acc, acc_phase, p.status, 4));
            if (!ok) break;
            tc_fence_after();
            const int n0 = it.n * BN;
            const int n_valid = min(BN, p.N - n0);
            const int m_first = (it.m * 2 + (int)rank) * BM + quarter * 32;
            const unsigned t_row = tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(acc * BN);
            epilogue_rows<BN, C::EPI_WARPS, C::OUT_BYTES>(t_row, m_first, lane, n0, n_valid, col_group, warp - 2, it.split, out_buf, out_tiles,
                                                          &map_y, y, p, act);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_block(acce0 + 8 * acc, 0));
            ++local;
        }
        if (lane == 0) tma_store_wait_all();
    }
    if (*reinterpret_cast<volatile int*>(p.status) != 0) drain_after_timeout();   // a wait ran out somewhere: let what is in flight land
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                    // neither block leaves while the other may still touch it
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, C::TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------ host side
// A [rows, cols] bfloat16 matrix with row stride ld (elements), moved in boxes of box_rows x box_cols:
// operand boxes are 64 wide with the 128-byte swizzle (out-of-range elements read as zero), result
// boxes 32 wide without swizzle (out-of-range elements are not written).
int tensor_map(CUtensorMap* out, const void* ptr, long long rows, long long cols, long long ld, int box_rows, int box_cols = BK) {
    const unsigned long long dims[2] = {(unsigned long long)cols, (unsigned long long)rows};
    const unsigned long long strides[1] = {(unsigned long long)ld * 2};
    const unsigned box[2] = {(unsigned)box_cols, (unsigned)box_rows};
    return ti_tensor_map_bf16(out, ptr, 2, dims, strides, box, box_cols == BK);
}

template <int BN, int MT>
int launch(void* y, const CUtensorMap& mw, const CUtensorMap& mx, const CUtensorMap& my, const Params& p, int sm_count, cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<BN, MT>::SMEM);
        if (e != cudaSuccess) return ti_fail("gemm_tcgen05: %s", cudaGetErrorString(e));
        configured = true;
    }
    const int tiles = p.m_tiles * p.n_tiles * p.splits;
    const int slots = sm_count * Cfg<BN, MT>::BLOCKS_PER_SM;
    const int grid = tiles < slots ? tiles : slots;
    ti_launch(gemm_tcgen05_kernel<BN, MT>, dim3(grid), dim3(Cfg<BN, MT>::THREADS), Cfg<BN, MT>::SMEM, stream, mw, mx, my, y, p);
    return ti_check_launch("gemm_tcgen05");
}

// How many pairs of blocks of the pair kernel the device holds at once (0: none, the kernel is not used).
int pair_clusters(int sm_count) {
    static int clusters = -1;
    if (clusters < 0) {
        clusters = 0;
        if (cudaFuncSetAttribute(gemm_tcgen05_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PairCfg::SMEM) == cudaSuccess) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(sm_count & ~1); cfg.blockDim = dim3(PairCfg::THREADS); cfg.dynamicSmemBytes = PairCfg::SMEM;
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, gemm_tcgen05_pair_kernel, &cfg) == cudaSuccess && n > 0) clusters = n;
        }
        cudaGetLastError();
    }
    return clusters;
}

int launch_pair(void* y, const CUtensorMap& mw, const CUtensorMap& mx, const CUtensorMap& my, const Params& p, cudaStream_t stream) {
    const int clusters = pair_clusters(0);
    const int tiles = p.m_tiles * p.n_tiles * p.splits;
    const int pairs = tiles < clusters ? tiles : clusters;
    ti_launch(gemm_tcgen05_pair_kernel, dim3(2 * pairs), dim3(PairCfg::THREADS), PairCfg::SMEM, stream, mw, mx, my, y, p);
    return ti_check_launch("gemm_tcgen05 (pairs)");
}

// Chooses the tile shape and kernel for one product. (Giving the rows of a ragged last wave to a second
// launch with smaller tiles was measured and is slower: the few tiles of a last wave run faster than
// those of a full one, with the memory system and the power budget to themselves.)
int gemm_dispatch(void* y, long long ldy, const void* x, long long ldx, const void* W, int n, int out, int in, int splits, int epilogue,
                  const XieluParams& act, int* status, cudaStream_t stream, int sm_count) {
    const int bn = n > 128 ? 256 : n > 64 ? 128 : n > 32 ? 64 : 32;
    Params p;
    p.N = n; p.K = in;
    // Wide token tiles (more than 128 tokens): two SMs share a tile of 256 weight rows x 256 tokens
    // (cta_group::2): per MMA each SM fills 32 KB of shared memory instead of 48 KB, both accumulator buffers
    // stay, so the epilogue (xIELU included) overlaps the next tile, and a stage of 128 of k means one barrier
    // round trip per 1,024 tensor-core cycles. Measured on 2048 tokens: up projection with xIELU 257 us
    // (296 us with 128-row blocks of one SM), q|k|v 72 us (82 us), o 49 us (55 us).
    // With a long k (the down projection) one block per SM with 256 weight rows, whose epilogue is not
    // overlapped but rare, is a little faster still (233 us against 239 us), where it needs fewer waves.
    int mt = 1;
    const long long n_t = (n + bn - 1) / bn;
    if (bn == 256 && splits <= 1 && in >= 8192) {
        const long long waves1 = (((out + BM - 1) / BM) * n_t + sm_count - 1) / sm_count;
        const long long waves2 = (((out + 2 * BM - 1) / (2 * BM)) * n_t + sm_count - 1) / sm_count;
        if (3 * waves2 < 2 * waves1) mt = 2;
    }
    // (A product of a few hundred tokens with few output rows has fewer tiles than there are SM pairs: it may come cut
    // over k, each slice a tile of its own, leaving 32-bit partial sums.)
    const bool pair = mt == 1 && bn == 256 && (splits <= 1 || (epilogue == EPI_PARTIAL && n > 256)) && out >= 2 * BM && pair_clusters(sm_count) > 0;
    if (pair) mt = 2;
    p.M = out;
    p.m_tiles = (out + mt * BM - 1) / (mt * BM);
    p.n_tiles = (int)n_t;
    p.k_blocks = pair ? (in + PairCfg::KB * BK - 1) / (PairCfg::KB * BK) : (in + BK - 1) / BK;     // the pair kernel's stages hold 128 of k
    p.splits = splits < 1 ? 1 : (splits > p.k_blocks ? p.k_blocks : splits);
    TI_REQUIRE(p.splits == 1 || epilogue == EPI_PARTIAL, "gemm_tcgen05: a split product leaves partial sums");
    p.ldy = ldy; p.epilogue = epilogue; p.act = act; p.status = status;
    CUtensorMap mw, mx, my;
    if (int rc = tensor_map(&mw, W, out, in, in, BM)) return rc;
    if (int rc = tensor_map(&mx, x, n, in, ldx, pair ? bn / 2 : bn)) return rc;   // a pair's blocks load half a token tile each
    // A step of a few tokens: all blocks would ask L2 for the same token lines at the same time, so each weight
    // tile walks its k range from a start of its own (a function of the tile alone: a token's result does not
    // depend on the step it is in). With many tokens the tiles of a row of blocks share lines on purpose.
    p.rotate = n <= 64;
    p.tma_out = bn >= 128 && (epilogue == EPI_NONE || epilogue == EPI_XIELU) && ldy % 8 == 0 && !((uintptr_t)y & 15);
    if (p.tma_out) {
        if (int rc = tensor_map(&my, y, n, out, ldy, 32, 32)) return rc;
    } else {
        my = mx;                   // not read
    }
    if (pair) return launch_pair(y, mw, mx, my, p, stream);
    switch (bn) {
        case 256: return mt == 2 ? launch<256, 2>(y, mw, mx, my, p, sm_count, stream) : launch<256, 1>(y, mw, mx, my, p, sm_count, stream);
        case 128: return launch<128, 1>(y, mw, mx, my, p, sm_count, stream);
        case 64: return launch<64, 1>(y, mw, mx, my, p, sm_count, stream);
        default: return launch<32, 1>(y, mw, mx, my, p, sm_count, stream);
    }
}

}  // namespace

// y: [n, ldy] bfloat16 (float32 for EPI_F32), or partial sums [splits, n, ldy] float32 for EPI_PARTIAL.
// `status` is a device word that must be zero; a non-zero value afterwards means a wait ran out.
// Returns 2 when the sizes are outside what the kernel takes (the caller then uses the plain product).
extern "C" int ti_gemm_tcgen05(void* y, long long ldy, const void* x, long long ldx, const void* W, int n, int out, int in,
                               int splits, int epilogue, float alpha_p, float alpha_n, float beta, float eps,
                               int* status, cudaStream_t stream) {
    if (n == 0) return 0;
    if (in % 8 != 0 || ldx % 8 != 0 || ((uintptr_t)W & 15) || ((uintptr_t)x & 15) || in < 8) {
        ti_fail("gemm_tcgen05 needs 16-byte aligned rows: in=%d, ldx=%lld", in, ldx);
        return 2;
    }
    TI_REQUIRE(epilogue >= 0 && epilogue <= 3, "gemm_tcgen05: unknown epilogue %d", epilogue);
    TI_REQUIRE(status != nullptr, "gemm_tcgen05: status word missing");
    static int sm_count = 0;
    if (!sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (sm_count <= 0) sm_count = 148;
    }
    return gemm_dispatch(y, ldy, x, ldx, W, n, out, in, splits, epilogue, XieluParams{alpha_p, alpha_n, beta, eps}, status, stream, sm_count);
}
